"""A tour of the public API (the reference's examples/library_usage.rs and basic.rs): tensors and autograd, modules,
one training loop, a checkpoint round trip through the reference's `rnnb` format, and the tokenizer.

    python examples/library_usage.py
"""
import _common
import torch

import rust_neural_network_b200 as nn_b200
from rust_neural_network_b200 import Adam, BpeTokenizer, Linear, MergeScoring, MSELoss, ReLU, Sequential, SimpleDataLoader, Tensor

dev = _common.device()
torch.manual_seed(0)
print("version", nn_b200.VERSION, "device", dev)

# 1. tensors: the reference's method names on top of torch.Tensor
a = Tensor.from_vec([1.0, 2.0, 3.0, 4.0], [2, 2])
b = Tensor.from_vec([5.0, 6.0, 7.0, 8.0], [2, 2])
print("A + B =", a.add(b).data().tolist(), " A @ B =", a.matmul(b).data().tolist())
w = Tensor.he([3, 2])
loss = w.matmul(a).sum()
loss.backward()
print("d(sum(W A))/dW =", w.grad().tolist())

# 2. a model, a forward pass, its parameters
model = Sequential().add(Linear(10, 32)).add(ReLU()).add(Linear(32, 16)).add(ReLU()).add(Linear(16, 5)).to_device(dev)
out = model(torch.randn(4, 10, device=dev))
print("output shape", tuple(out.shape), "parameter tensors", len(model.parameters()))

# 3. a training loop written by hand
opt, loss_fn = Adam(model.parameters(), lr=0.01), MSELoss("mean")
loader = SimpleDataLoader(torch.randn(32, 10), torch.randn(32, 5), 8)
for epoch in range(5):
    total = 0.0
    for bx, by in loader:
        opt.zero_grad()
        l = loss_fn(model(bx.to(dev)), by.to(dev))
        l.backward()
        opt.step()
        total += float(l)
    print(f"epoch {epoch}  mean batch loss {total / len(loader):.4f}")

# 4. checkpoint: bytes in the reference's format, loadable by either implementation
blob = nn_b200.save_model(model)
clone = Sequential().add(Linear(10, 32)).add(ReLU()).add(Linear(32, 16)).add(ReLU()).add(Linear(16, 5)).to_device(dev)
nn_b200.load_model(clone, blob)
x = torch.randn(2, 10, device=dev)
assert torch.allclose(model(x).float(), clone(x).float(), atol=1e-5)
print("checkpoint bytes", len(blob), "- reloaded model agrees")

# 5. byte-level BPE
tok = BpeTokenizer.train("the quick brown fox jumps over the lazy dog. the dog barks. " * 20, 300, MergeScoring.Frequency)
ids = tok.encode("the quick dog")
print("tokens", ids, "->", repr(tok.decode(ids)))
