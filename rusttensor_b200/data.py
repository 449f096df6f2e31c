"""The data path either side of the training step (src/data.rs): ``load_csv`` and random batches.

``load_csv`` follows src/data.rs:13-123: no header row, first column the label (an integer 0..9), the remaining columns
features that are divided by 255; labels become one-hot rows of 10 classes; the same checks in the same order with the same
error variants.  Batches come from ``engine.get_random_batch`` / ``engine.get_batch`` (src/data.rs:125-209), which gather
the rows with the backend: the data set stays on the device and only the row numbers travel.
"""
import csv

import numpy as np

from .frontend import ERROR_KINDS, EngineError

NUM_CLASSES = 10  # "MNIST specific" in the reference (src/data.rs:22)
_INVALID_OPERATION = 4
_CSV_ERROR = 17
ERROR_KINDS.setdefault(_CSV_ERROR, "CsvError")


def parse_csv(path):
    """(features [n, f] float32 in [0, 1], one-hot labels [n, 10] float32) as numpy arrays."""
    feats, labels, n_feat = [], [], None
    try:
        f = open(path, newline="")
    except OSError as e:
        raise EngineError(_CSV_ERROR, str(e)) from e
    with f:
        for row_idx, rec in enumerate(csv.reader(f)):
            if len(rec) == 0:
                continue  # the csv crate skips empty lines as well
            label_str = rec[0]
            try:
                label = np.float32(label_str.strip()) if label_str.strip() else np.float32("nan")
                label = float(label)
                if label != label:
                    raise ValueError("nan")
            except ValueError as e:
                raise EngineError(_INVALID_OPERATION, f"Invalid label format at row {row_idx}: '{label_str}' - {e}") from e
            if not (0.0 <= label < NUM_CLASSES) or label != int(label):
                raise EngineError(_INVALID_OPERATION,
                                  f"Invalid label value at row {row_idx}: {label}. Expected integer 0-{NUM_CLASSES - 1}.")
            cur = []
            for col_idx, s in enumerate(rec[1:]):
                try:
                    cur.append(float(np.float32(s.strip())))
                except ValueError as e:
                    raise EngineError(_INVALID_OPERATION,
                                      f"Invalid feature format at row {row_idx}, column {col_idx + 1}: '{s}' - {e}") from e
            if n_feat is None:
                if not cur:
                    raise EngineError(_INVALID_OPERATION, "Row with label but no features found.")
                n_feat = len(cur)
            elif len(cur) != n_feat:
                raise EngineError(_INVALID_OPERATION,
                                  f"Inconsistent number of features at row {row_idx}. Expected {n_feat}, found {len(cur)}")
            labels.append(int(label))
            feats.append(cur)
    n = len(labels)
    x = (np.asarray(feats, dtype=np.float32).reshape(n, n_feat or 0) / np.float32(255.0)).astype(np.float32)
    y = np.zeros((n, NUM_CLASSES), dtype=np.float32)
    y[np.arange(n), labels] = 1.0
    return x, y


def load_csv(engine, path):
    """``load_csv::<B>(path)`` (src/data.rs:13-123): two tensors on ``engine``, neither requiring a gradient.  An empty file
    gives tensors of shape [0, 0] and [0, 10]."""
    x, y = parse_csv(path)
    return engine.tensor(x, x.shape, False), engine.tensor(y, y.shape, False)
