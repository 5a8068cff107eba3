"""Interactive session (rust-nn src/interactive.rs): `Session`, `run_repl`, `process_command`, `sparkline`.

One dispatcher (`Session.execute`) serves both the REPL and the programmatic `process_command`; it
returns the text instead of printing it. Commands: tensor, model, data, train, predict, info, device,
help, exit - the reference's set plus `device cpu|cuda` (models and data then live on the GPU and
`train` runs the full-batch loop there).
"""
from __future__ import annotations

import sys
from typing import List, Optional

import torch

from . import data as D
from . import nn
from .loss import MSELoss
from .optim import Adam

BANNER = """
  +-------------------------------------------+
  |   rust-nn (B200) Interactive Session      |
  |   tcgen05 kernels behind a line REPL      |
  +-------------------------------------------+
  Type 'help' for commands. 'exit' to quit.
"""

HELP = """
  Commands:
    tensor randn|zeros|ones <dims...>   Create a tensor and print it

    model new                     Start a new Sequential model
    model add linear <in> <out>   Add a Linear(in, out) layer with bias
    model add relu|sigmoid|tanh|gelu|silu   Add an activation
    model summary                 Print model architecture and param count

    data csv|tsv|jsonl <path>     Load a file
    data hf <dataset> <split> <n> Load n rows from HuggingFace Hub (or its local cache)
    data synthetic <n> <f> <c>    Synthetic classification data (n samples, f features, c classes)
    data regression <n> <f>       Synthetic regression data
    data columns                  List dataset columns
    data head <n>                 Show first n rows
    data target <column>          Set the target/label column
    data features <col1> <col2>   Set feature columns (space-separated)

    device cpu|cuda               Where models and batches live
    train <epochs> <lr>           Train the model on the loaded dataset (Adam, MSE)
    predict <row>                 Run inference on a specific row
    info                          Show current session state
    exit                          Quit
"""

_BLOCKS = "▁▂▃▄▅▆▇█"


def sparkline(values) -> str:
    values = list(values)
    if not values:
        return ""
    lo, hi = min(values), max(values)
    if hi - lo < 1e-12:
        return _BLOCKS[7] * len(values)
    return "".join(_BLOCKS[min(int((v - lo) / (hi - lo) * 7.0 + 0.5), 7)] for v in values)


class Session:
    def __init__(self):
        self.model: Optional[nn.Sequential] = None
        self.model_input_dim: Optional[int] = None
        self.model_output_dim: Optional[int] = None
        self.dataset: Optional[D.Dataset] = None
        self.feature_columns: List[str] = []
        self.target_column: Optional[str] = None
        self.device = torch.device("cpu")
        self.losses: List[float] = []

    @staticmethod
    def new() -> "Session":
        return Session()

    # ---- command handlers; each returns the text to show
    def _tensor(self, a: List[str]) -> str:
        if not a:
            return "Usage: tensor randn|zeros <dims...>"
        dims = [int(s) for s in a[1:] if s.isdigit()]
        if not dims:
            return "Error: provide at least one dimension"
        make = {"randn": torch.randn, "zeros": torch.zeros, "ones": torch.ones}.get(a[0])
        if make is None:
            return f"Unknown tensor command: {a[0]}"
        from .tensor import Tensor
        return str(Tensor(make(*dims)))

    def _model(self, a: List[str]) -> str:
        if not a:
            return "Usage: model new|add|summary"
        if a[0] == "new":
            self.model, self.model_input_dim, self.model_output_dim = nn.Sequential(), None, None
            return "New model created: started a new Sequential model."
        if a[0] == "add":
            if self.model is None:
                return "No model. Run 'model new' first."
            if len(a) < 2:
                return "Usage: model add linear|relu|sigmoid|tanh ..."
            if a[1] == "linear":
                if len(a) < 4:
                    return "Usage: model add linear <in_features> <out_features>"
                in_f = int(a[2]) if a[2].isdigit() else 0
                out_f = int(a[3]) if a[3].isdigit() else 0
                if in_f == 0 or out_f == 0:
                    return "Error: invalid dimensions"
                if self.model_input_dim is None:
                    self.model_input_dim = in_f
                self.model_output_dim = out_f
                layer = nn.Linear(in_f, out_f, True)
                if self.device.type == "cuda":
                    layer.to_device(self.device)
                self.model.add(layer)
                return f"Added Linear({in_f} -> {out_f})"
            acts = {"relu": nn.ReLU, "sigmoid": nn.Sigmoid, "tanh": nn.Tanh, "gelu": nn.GELU, "silu": nn.SiLU}
            if a[1] in acts:
                self.model.add(acts[a[1]]())
                return f"Added {acts[a[1]].__name__}"
            return f"Unknown layer: {a[1]}"
        if a[0] == "summary":
            if self.model is None:
                return "No model loaded."
            ps = self.model.parameters()
            out = f"\n  Model: Sequential\n  Parameters: {len(ps)} tensors, {sum(p.numel() for p in ps)} total elements"
            if self.model_input_dim is not None and self.model_output_dim is not None:
                out += f"\n  Input dim: {self.model_input_dim}, Output dim: {self.model_output_dim}"
            return out
        return f"Unknown model command: {a[0]}"

    def _set_dataset(self, ds: D.Dataset) -> str:
        self.dataset = ds
        return ds.summary()

    def _data(self, a: List[str]) -> str:
        if not a:
            return "Usage: data csv|tsv|jsonl|hf|synthetic|regression|columns|head|features|target"
        try:
            if a[0] in ("csv", "tsv", "jsonl") and len(a) >= 2:
                return self._set_dataset({"csv": D.load_csv, "tsv": D.load_tsv, "jsonl": D.load_jsonl}[a[0]](a[1]))
            if a[0] == "hf" and len(a) >= 4:
                n = int(a[3]) if a[3].isdigit() else 100
                return f"Loading from HuggingFace: {a[1]}/{a[2]} ({n} rows)...\n" + self._set_dataset(D.load_huggingface(a[1], a[2], n))
        except D.DataError as e:
            return f"Error: {e}"
        if a[0] == "synthetic" and len(a) >= 3:
            n = int(a[1]) if a[1].isdigit() else 100
            f = int(a[2]) if a[2].isdigit() else 4
            c = int(a[3]) if len(a) > 3 and a[3].isdigit() else 3
            out = self._set_dataset(D.make_classification(n, f, c))
            self.feature_columns, self.target_column = [f"f{j}" for j in range(f)], "label"
            return out
        if a[0] == "regression" and len(a) >= 3:
            n = int(a[1]) if a[1].isdigit() else 100
            f = int(a[2]) if a[2].isdigit() else 4
            out = self._set_dataset(D.make_regression(n, f))
            self.feature_columns, self.target_column = [f"f{j}" for j in range(f)], "target"
            return out
        if a[0] == "columns":
            if self.dataset is None:
                return "No dataset loaded."
            lines = []
            for name in sorted(self.dataset.columns):
                col = self.dataset.columns[name]
                mark = " [feature]" if name in self.feature_columns else " [target]" if name == self.target_column else ""
                lines.append(f"  {name}: {'f32' if col.is_numeric() else 'str'}{mark}")
            return "\n".join(lines)
        if a[0] == "head":
            if self.dataset is None:
                return "No dataset loaded."
            n = int(a[1]) if len(a) > 1 and a[1].isdigit() else 5
            return self.dataset.head(n).summary()
        if a[0] == "features":
            self.feature_columns = list(a[1:])
            return f"Feature columns: {self.feature_columns}"
        if a[0] == "target" and len(a) >= 2:
            self.target_column = a[1]
            return f"Target column: {a[1]}"
        return "Unknown data command or missing arguments. Type 'help'."

    def _device(self, a: List[str]) -> str:
        want = a[0] if a else "cpu"
        if want.startswith("cuda") and not torch.cuda.is_available():
            return "Error: no CUDA device available"
        self.device = torch.device(want)
        if self.model is not None:
            self.model.to_device(self.device)
        return f"Device: {self.device}"

    def _train(self, a: List[str]) -> str:
        epochs = int(a[0]) if a and a[0].isdigit() else 10
        try:
            lr = float(a[1]) if len(a) > 1 else 0.01
        except ValueError:
            lr = 0.01
        if self.model is None or self.dataset is None:
            return "Need both a model and a dataset. Use 'model new' and 'data ...' first."
        if not self.feature_columns or self.target_column is None:
            return "Set feature and target columns first. Use 'data features ...' and 'data target ...'."
        x = self.dataset.to_tensor(self.feature_columns, self.device)
        y = self.dataset.to_tensor([self.target_column], self.device)
        opt, loss_fn = Adam(self.model.parameters(), lr=lr), MSELoss()
        out = [f"\n  Training: {epochs} epochs, lr={lr}", "  " + "-" * 50]
        dev_losses = []
        for _ in range(epochs):
            opt.zero_grad()
            loss = loss_fn(self.model(x), y)
            loss.backward()
            opt.step()
            dev_losses.append(loss.detach().float() / max(x.numel(), 1))
        losses = torch.stack(dev_losses).cpu().tolist() if dev_losses else []      # one read-back for the whole run
        for e in range(len(losses)):
            out.append(f"  Epoch {e + 1:>3}: loss = {losses[e]:>10.4f} {sparkline(losses[: e + 1])}")
        self.losses = losses
        out += ["  " + "-" * 50, f"  Training complete. Final loss: {losses[-1] if losses else 0.0:.4f}\n"]
        return "\n".join(out)

    def _predict(self, a: List[str]) -> str:
        row = int(a[0]) if a and a[0].isdigit() else 0
        if self.model is None or self.dataset is None:
            return "Need both a model and a dataset."
        x = self.dataset.head(row + 1).to_tensor(self.feature_columns, self.device)
        with torch.no_grad():
            y = self.model(x).float().cpu()
        return f"  Prediction for row {row}: {[round(v, 6) for v in y[min(row, y.shape[0] - 1)].tolist()]}"

    def _info(self) -> str:
        out = ["\n  Session state:", f"    Model: {'loaded' if self.model is not None else 'none'}",
               f"    Dataset: {'loaded' if self.dataset is not None else 'none'}", f"    Device: {self.device}"]
        if self.feature_columns:
            out.append(f"    Features: {self.feature_columns}")
        if self.target_column:
            out.append(f"    Target: {self.target_column}")
        return "\n".join(out) + "\n"

    def execute(self, line: str) -> Optional[str]:
        """Runs one command line; returns its output, or None for exit/quit."""
        parts = line.split()
        if not parts:
            return ""
        cmd, args = parts[0], parts[1:]
        if cmd in ("help", "?", "h"):
            return HELP
        if cmd in ("exit", "quit", "q"):
            return None
        handlers = {"tensor": self._tensor, "model": self._model, "data": self._data, "train": self._train,
                    "predict": self._predict, "device": self._device}
        if cmd == "info":
            return self._info()
        if cmd in handlers:
            return handlers[cmd](args)
        return f"Unknown command: '{cmd}'. Type 'help' for available commands."


def process_command(session: Session, command: str) -> str:
    """Programmatic entry (src/interactive.rs:485-540). `info` answers in the compact form
    `model: true|false, dataset: true|false`; unknown commands and exit give an empty string."""
    parts = command.split()
    if not parts:
        return ""
    if parts[0] == "info":
        return f"model: {str(session.model is not None).lower()}, dataset: {str(session.dataset is not None).lower()}"
    if parts[0] not in ("tensor", "model", "data", "train", "predict", "device"):
        return ""
    return session.execute(command) or ""


def run_repl(stdin=None, stdout=None) -> None:
    stdin, stdout = stdin or sys.stdin, stdout or sys.stdout
    session = Session()
    stdout.write(BANNER + "\n")
    while True:
        stdout.write("rust-nn> ")
        stdout.flush()
        line = stdin.readline()
        if not line:
            break
        line = line.strip()
        if not line:
            continue
        out = session.execute(line)
        if out is None:
            stdout.write("Goodbye!\n")
            break
        stdout.write(out + "\n")
