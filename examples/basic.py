"""Tensor operations, activations, a small network and broadcasting through the reference-shaped API (the reference's
examples/basic.rs, section by section): `Tensor.from_vec`, `.add / .mul / .matmul / .reshape / .transpose`, the
functional activations, `Sequential.new().add(Linear.new(...)).add(ReLU)`.

    python examples/basic.py
"""
import _common  # noqa: F401
import torch

from rust_neural_network_b200.activations import relu, sigmoid, softmax
from rust_neural_network_b200.nn import Linear, ReLU, Sequential
from rust_neural_network_b200.tensor import Tensor

torch.manual_seed(0)
print("1. Tensor operations")
print("zeros", Tensor.zeros([2, 3]).data().tolist())
print("ones ", Tensor.ones([2, 3]).data().tolist())
a = Tensor.from_vec([1.0, 2.0, 3.0, 4.0], [2, 2])
b = Tensor.from_vec([5.0, 6.0, 7.0, 8.0], [2, 2])
print("A + B ", a.add(b).data().tolist())
print("A * B ", a.mul(b).data().tolist())
print("A @ B ", a.matmul(b).data().tolist())
flat = Tensor.from_vec([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], [2, 3])
print("reshape [2,3] -> [3,2]", flat.reshape([3, 2]).data().tolist())
print("A transposed", a.transpose().data().tolist())
print(f"sum {float(a.sum().data()):.4f}  mean {a.mean():.4f}  max {a.max():.4f}")
assert a.matmul(b).data().tolist() == [[19.0, 22.0], [43.0, 50.0]]

print("\n2. Activation functions")
x = Tensor.from_vec([-2.0, -1.0, 0.0, 1.0, 2.0], [5])
print("relu   ", relu(x).data().tolist())
print("sigmoid", [round(v, 4) for v in sigmoid(x).data().tolist()])
sm = softmax(Tensor.from_vec([1.0, 2.0, 3.0], [3]))
print("softmax([1,2,3])", [round(v, 4) for v in sm.data().tolist()], "sum", round(float(sm.sum().data()), 6))

print("\n3. Neural network")
model = Sequential.new().add(Linear.new(10, 32, True)).add(ReLU).add(Linear.new(32, 16, True)).add(ReLU).add(Linear.new(16, 5, True))
inp = Tensor.randn([4, 10])
out = model.forward(inp)
print("input shape", inp.shape(), "output shape", out.shape())
print("first sample", [round(out.get([0, i]), 4) for i in range(5)])
params = model.parameters()
print(len(params), "parameter tensors:", [list(p.shape) for p in params])
assert out.shape() == [4, 5] and len(params) == 6

print("\n4. Broadcasting")
matrix = Tensor.from_vec([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], [2, 3])
bias = Tensor.from_vec([0.1, 0.2, 0.3], [3])
print("matrix + bias", [[round(v, 2) for v in row] for row in matrix.add(bias).data().tolist()])
