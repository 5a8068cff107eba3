"""XOR with a 2-8-1 MLP (the reference's examples/xor.rs): Sequential, Tanh, MSELoss, Adam, Trainer.

    python examples/xor.py
"""
import _common
import torch

from rust_neural_network_b200 import Adam, Linear, MSELoss, Sequential, SimpleDataLoader, Tanh, Trainer

dev = _common.device()
torch.manual_seed(0)
x = torch.tensor([[0.0, 0.0], [0.0, 1.0], [1.0, 0.0], [1.0, 1.0]])
y = torch.tensor([[0.0], [1.0], [1.0], [0.0]])
model = Sequential().add(Linear(2, 8)).add(Tanh()).add(Linear(8, 1)).to_device(dev)
trainer = Trainer(model, Adam(model.parameters(), lr=0.05), MSELoss())
loader = SimpleDataLoader(x, y, 4)
for epoch in range(400):
    loss = trainer.train_epoch(loader)
    if epoch % 100 == 0:
        print(f"epoch {epoch:3d}  loss {loss:.5f}")
pred = model(x.to(dev)).detach().cpu().flatten().tolist()
print("final loss", round(loss, 5), "predictions", [round(p, 3) for p in pred])
assert loss < 0.1
