"""Checkpoint / resume of a training run, interoperable with the reference's tensor files.

The reference saves one tensor per file as the serde_json image of ``SerializableTensor``
(src/tensor.rs:38-47, 130-165, 444-502)::

    {"data": [f32 ...], "shape": [usize ...], "grad": null | [f32 ...], "requires_grad": bool, "device": "Cpu" | {"Cuda": id}}

``save_tensor`` / ``load_tensor`` write and read exactly that file.  ``save_checkpoint`` / ``load_checkpoint`` put a
whole data-parallel trainer (parameters, the optimizer's state tensors and its step counter) into one JSON document whose
tensor entries have the same layout, so each of them can be cut out and read by the reference on its own.

Floats are written with enough digits to come back bit for bit (serde_json writes the shortest such form; any decimal
that rounds to the same f32 loads identically on both sides).  Non-finite values become ``null`` as in serde_json and are
read back as NaN.
"""
import json
import math

import numpy as np

FORMAT = "rusttensor-b200-checkpoint"
VERSION = 1
_OPTIMIZERS = {0: "none", 1: "adam", 2: "momentum_sgd"}


def _floats(a):
    out = np.asarray(a, dtype=np.float32).ravel().tolist()
    if not all(map(math.isfinite, out)):
        out = [v if math.isfinite(v) else None for v in out]
    return out


def _array(values, shape):
    a = np.array([np.nan if v is None else v for v in values], dtype=np.float32)
    n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
    if a.size != n:
        raise ValueError(f"tensor entry holds {a.size} values for shape {list(shape)}")
    return a.reshape(shape)


def tensor_record(data, grad=None, requires_grad=False, device=None):
    """The reference's ``SerializableTensor`` as a dict; ``device`` None / "cpu" -> "Cpu", an int -> {"Cuda": id}."""
    data = np.asarray(data, dtype=np.float32)
    return {"data": _floats(data), "shape": [int(s) for s in data.shape], "grad": None if grad is None else _floats(grad),
            "requires_grad": bool(requires_grad), "device": "Cpu" if device in (None, "cpu", "Cpu") else {"Cuda": int(device)}}


def record_arrays(rec):
    """(data, grad or None, requires_grad) of a ``SerializableTensor`` dict."""
    shape = tuple(int(s) for s in rec["shape"])
    grad = rec.get("grad")
    return _array(rec["data"], shape), None if grad is None else _array(grad, shape), bool(rec.get("requires_grad", False))


def save_tensor(tensor, path, device=0):
    """``Tensor::save_to_file`` (src/tensor.rs:444-456): one engine tensor (with its gradient, if any) as a reference file."""
    g = tensor.grad
    with open(path, "w") as f:
        json.dump(tensor_record(tensor.numpy(), None if g is None else g.numpy(), tensor.requires_grad, device), f, separators=(",", ":"))


def load_tensor(engine, path):
    """``Tensor::load_from_file`` (src/tensor.rs:481-502): a new tensor on ``engine`` from a reference file."""
    with open(path) as f:
        data, grad, rg = record_arrays(json.load(f))
    t = engine.tensor(data, data.shape, rg)
    if grad is not None:
        t.set_grad(engine.tensor(grad, grad.shape))
    return t


def save_checkpoint(trainer, path, device=0):
    """Parameters, optimizer state and step counter of a ``DataParallelTrainer`` (all ranks hold the same values: rank 0
    saves).  Synchronises with the device."""
    kind = trainer.optimizer_kind
    n = len(trainer.params)
    doc = {"format": FORMAT, "version": VERSION, "optimizer": _OPTIMIZERS[kind], "t": trainer.step_count,
           "params": [tensor_record(p.numpy(), requires_grad=True, device=device) for p in trainer.params],
           "state1": [tensor_record(trainer.state(0, i).numpy(), device=device) for i in range(n)] if kind in (1, 2) else [],
           "state2": [tensor_record(trainer.state(1, i).numpy(), device=device) for i in range(n)] if kind == 1 else []}
    with open(path, "w") as f:
        json.dump(doc, f, separators=(",", ":"))


def load_checkpoint(trainer, path):
    """Restores what ``save_checkpoint`` wrote into a trainer of the same workload; raises ``ValueError`` when the file does
    not fit (format, optimizer, number or shapes of the tensors)."""
    with open(path) as f:
        doc = json.load(f)
    if doc.get("format") != FORMAT or doc.get("version") != VERSION:
        raise ValueError(f"{path}: not a {FORMAT} v{VERSION} file")
    kind = trainer.optimizer_kind
    if doc.get("optimizer") != _OPTIMIZERS[kind]:
        raise ValueError(f"{path}: saved for optimizer {doc.get('optimizer')!r}, the trainer uses {_OPTIMIZERS[kind]!r}")
    params = [record_arrays(r)[0] for r in doc["params"]]
    if len(params) != len(trainer.params):
        raise ValueError(f"{path}: {len(params)} parameters, the trainer has {len(trainer.params)}")
    for i, (t, a) in enumerate(zip(trainer.params, params)):
        if tuple(t.shape) != a.shape:
            raise ValueError(f"{path}: parameter {i} has shape {a.shape}, the trainer expects {tuple(t.shape)}")
    for t, a in zip(trainer.params, params):
        t.update_from_host(a)
    for which, key in ((0, "state1"), (1, "state2")):
        for i, r in enumerate(doc.get(key, [])):
            trainer.set_state(which, i, record_arrays(r)[0])
    trainer.step_count = int(doc["t"])
