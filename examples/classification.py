"""Three-class classification on a synthetic dataset (the reference's examples/classification.rs): `make_classification`,
`train_test_split`, a ReLU MLP, cross-entropy on one-hot targets, accuracy on the held-out rows.

    python examples/classification.py
"""
import _common
import torch

from rust_neural_network_b200 import Adam, CrossEntropyLoss, Linear, ReLU, Sequential, SimpleDataLoader, Trainer, make_classification

dev = _common.device()
torch.manual_seed(1)
ds = make_classification(600, 8, 3)
train, test = ds.train_test_split(0.8)
features = [f"f{j}" for j in range(8)]


def tensors(d):
    return d.to_tensor(features), d.to_tensor(["label"]).flatten().long()


xtr, ytr = tensors(train)
xte, yte = tensors(test)
model = Sequential().add(Linear(8, 32)).add(ReLU()).add(Linear(32, 3)).to_device(dev)
trainer = Trainer(model, Adam(model.parameters(), lr=0.01), CrossEntropyLoss())
loader = SimpleDataLoader(xtr, torch.nn.functional.one_hot(ytr, 3).float(), 32)
for epoch in range(30):
    loss = trainer.train_epoch(loader)
acc = float((model(xte.to(dev)).argmax(-1).cpu() == yte).float().mean())
print(f"train loss {loss:.4f}  test accuracy {acc:.3f}")
assert acc > 0.6
