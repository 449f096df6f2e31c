"""Data-parallel training step on the CUDA backend (one process per GPU).

forward + backward are replayed from a CUDA graph, the flat gradient buffer is summed
with one NCCL all-reduce, and one fused multi-tensor kernel applies the optimizer
(with the 1/world scale and the optional gradient clip folded in).
"""
import ctypes as C

import numpy as np

from .frontend import Tensor, EngineError, _i64, _f64

_f32p = C.POINTER(C.c_float)


class DataParallelTrainer:
    def __init__(self, config, dims, rank=0, world=1, nccl_id=None, device=None):
        from . import engine

        self.engine = engine(device)
        self.host = self.engine.lib
        self.rank, self.world = rank, world
        idbuf = (C.c_uint8 * 128)(*(nccl_id if nccl_id is not None else [0] * 128))
        out = C.c_int64(0)
        self._call("dp_create", C.c_int(config), _i64(dims), C.c_int(len(dims)), C.c_int(rank), C.c_int(world), idbuf,
                   C.byref(out))
        self.handle = out.value
        n = C.c_int(0)
        self._call("dp_num_params", C.c_int64(self.handle), C.byref(n))
        self.params = [self._tensor("dp_param", i) for i in range(n.value)]
        self.inputs = []
        i = 0
        while True:
            try:
                self.inputs.append(self._tensor("dp_input", i))
            except EngineError:
                break
            i += 1
        self._pinned = []
        for i, t in enumerate(self.inputs):
            p = _f32p()
            self._call("dp_pinned_input", C.c_int64(self.handle), C.c_int(i), C.byref(p))
            self._pinned.append(np.ctypeslib.as_array(p, shape=t.shape))

    def _call(self, name, *args):
        self.engine._call(name, *args)

    def _tensor(self, fn, i, *extra):
        h = C.c_int64(0)
        self._call(fn, C.c_int64(self.handle), *extra, C.c_int(i), C.byref(h))
        return Tensor(self.engine, h.value)

    def __del__(self):
        try:
            self._call("dp_free", C.c_int64(self.handle))
        except Exception:
            pass

    @staticmethod
    def unique_id():
        """A fresh NCCL id (rank 0 creates it and sends the 128 bytes to every rank)."""
        from . import load_library

        buf = (C.c_uint8 * 128)()
        rc = load_library().rt_dp_unique_id(buf)
        if rc != 0:
            raise RuntimeError(f"rt_dp_unique_id failed with status {rc}")
        return bytes(buf)

    def set_hyper(self, *hp):
        self._call("dp_set_hyper", C.c_int64(self.handle), _f64(hp), C.c_int(len(hp)))

    @property
    def optimizer_kind(self):
        """0: none, 1: Adam, 2: MomentumSGD."""
        k = C.c_int(0)
        self._call("dp_optimizer_kind", C.c_int64(self.handle), C.byref(k))
        return k.value

    @property
    def peer_wait_ns(self):
        """Time this rank has spent waiting for its peers' gradients in the exchange over peer memory (synchronises)."""
        n = C.c_int64(0)
        self._call("dp_peer_wait_ns", C.c_int64(self.handle), C.byref(n))
        return n.value

    def trace(self):
        """RT_B200_DP_TRACE=1: GPU time stamps (ns) of the last step: [start, forward done, backward done, packed + signalled,
        peers complete, -, optimizer done]; zeros where a stamp does not exist in this mode."""
        out = (C.c_int64 * 8)()
        self._call("dp_trace", C.c_int64(self.handle), out, C.c_int(8))
        return list(out)

    @property
    def flat_len(self):
        """Floats in the flat gradient buffer (every tensor's start padded to 16 bytes): equal on all ranks of a job."""
        n = C.c_int64(0)
        self._call("dp_flat_len", C.c_int64(self.handle), C.byref(n))
        return n.value

    @property
    def step_count(self):
        """Number of optimizer steps taken (Adam's ``t``)."""
        t = C.c_int64(0)
        self._call("dp_get_step", C.c_int64(self.handle), C.byref(t))
        return t.value

    @step_count.setter
    def step_count(self, t):
        self._call("dp_set_step", C.c_int64(self.handle), C.c_int64(int(t)))

    def set_state(self, which, i, array):
        a = np.require(array, dtype=np.float32, requirements='C')
        self._call("dp_set_state", C.c_int64(self.handle), C.c_int(which), C.c_int(i), a.ctypes.data_as(_f32p), C.c_int64(a.size))

    def state(self, which, i):
        return self._tensor("dp_state", i, C.c_int(which))

    def pinned_input(self, i):
        """numpy view of the pinned host staging buffer of input ``i``."""
        return self._pinned[i]

    def _ptrs(self, arrays):
        keep = [np.require(a, dtype=np.float32, requirements='C') for a in arrays]
        arr = (_f32p * len(keep))(*[a.ctypes.data_as(_f32p) for a in keep])
        return keep, arr

    def step_eager(self, arrays):
        keep, arr = self._ptrs(arrays)
        loss = C.c_float(0)
        self._call("dp_step_eager", C.c_int64(self.handle), arr, C.c_int(len(keep)), C.byref(loss))
        return loss.value

    def capture(self):
        self._call("dp_capture", C.c_int64(self.handle))

    def step(self, arrays=None, pinned=False):
        """Enqueues one step.  ``arrays``: host inputs (copied through pinned staging), or None to
        reuse the inputs resident on the device; ``pinned=True`` takes the data already written
        into ``pinned_input(i)``."""
        if pinned:
            arr = (_f32p * len(self._pinned))(*[a.ctypes.data_as(_f32p) for a in self._pinned])
            self._call("dp_step_graph", C.c_int64(self.handle), arr, C.c_int(len(self._pinned)), C.c_int(1))
        elif arrays is None:
            self._call("dp_step_graph", C.c_int64(self.handle), None, C.c_int(0), C.c_int(0))
        else:
            keep, arr = self._ptrs(arrays)
            self._call("dp_step_graph", C.c_int64(self.handle), arr, C.c_int(len(keep)), C.c_int(0))

    def last_loss(self):
        loss = C.c_float(0)
        self._call("dp_last_loss", C.c_int64(self.handle), C.byref(loss))
        return loss.value

    # ---- gradient exchange fused into the optimizer step over peer memory (world > 1) ----
    def fused_export(self):
        """192 bytes: the IPC handles of this rank's two flat gradient buffers and of its flag array."""
        buf = (C.c_uint8 * 192)()
        self._call("dp_fused_export", C.c_int64(self.handle), buf)
        return bytes(buf)

    def fused_connect(self, all_handles):
        """``all_handles``: the 192-byte blobs of every rank, concatenated in rank order."""
        data = bytes(all_handles)
        assert len(data) == 192 * self.world
        buf = (C.c_uint8 * len(data)).from_buffer_copy(data)
        self._call("dp_fused_connect", C.c_int64(self.handle), buf)

    def connect_peers(self, dist):
        """Sets the fused exchange up through a ``torch.distributed`` process group.  Every rank calls it and every rank
        gets the same answer: True when all ranks are connected; False when any rank failed (the trainer must then be
        discarded and a new one used with the NCCL exchange).  All collectives run on every rank whatever fails."""
        import torch

        device = "cuda" if dist.get_backend() == "nccl" else "cpu"
        ok, blob = 1, bytes(192)
        try:
            blob = self.fused_export()
        except Exception as e:  # noqa: BLE001
            ok, self.peer_error = 0, str(e)
        mine = torch.tensor(list(blob) + [ok], dtype=torch.uint8, device=device)
        parts = [torch.zeros_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine)
        rows = [bytes(p.cpu().tolist()) for p in parts]
        ok = min(r[192] for r in rows)
        if ok:
            try:
                self.fused_connect(b"".join(r[:192] for r in rows))
            except Exception as e:  # noqa: BLE001
                ok, self.peer_error = 0, str(e)
        flag = torch.tensor([ok], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return bool(flag.item())

    # ---- pipelined steps: the upload of step i+1 overlaps the device work of step i ----
    def pipeline_buffer(self, i):
        """numpy view of the pinned host buffer to fill with input ``i`` of the NEXT pipelined step
        (two buffers alternate; the call waits until the copy that last read this one has finished)."""
        p = _f32p()
        self._call("dp_pipeline_buffer", C.c_int64(self.handle), C.c_int(i), C.byref(p))
        return np.ctypeslib.as_array(p, shape=tuple(self.inputs[i].shape))

    def step_pipelined(self):
        """Enqueues one step from the pipeline buffers and returns the loss of the previous pipelined
        step (None for the first one): the host never waits for the step it has just enqueued."""
        loss, has = C.c_float(0), C.c_int(0)
        self._call("dp_step_pipelined", C.c_int64(self.handle), C.byref(loss), C.byref(has))
        return loss.value if has.value else None

    # ---- steps fed from a data set resident on the device (src/data.rs:125-209 without the host round trip) ----
    def attach_dataset(self, arrays):
        """``arrays``: one host array per input with the samples along axis 0 (same number of rows each); uploaded once."""
        keep, arr = self._ptrs([np.asarray(a, dtype=np.float32).reshape(len(a), -1) for a in arrays])
        rows = keep[0].shape[0]
        assert all(a.shape[0] == rows for a in keep)
        self._call("dp_attach_dataset", C.c_int64(self.handle), arr, C.c_int(len(keep)), C.c_int64(rows))

    def step_dataset(self, indices):
        """Enqueues one step on rows ``indices`` of the attached data set (only the indices are uploaded; the batch is gathered on
        the device) and returns the loss of the previous such step (None for the first)."""
        idx = np.require(indices, dtype=np.int64, requirements='C')
        loss, has = C.c_float(0), C.c_int(0)
        self._call("dp_step_dataset", C.c_int64(self.handle), idx.ctypes.data_as(C.POINTER(C.c_int64)), C.c_int64(idx.size),
                   C.byref(loss), C.byref(has))
        return loss.value if has.value else None

    def pipeline_flush(self):
        """Waits for the last pipelined step and returns its loss."""
        loss = C.c_float(0)
        self._call("dp_pipeline_flush", C.c_int64(self.handle), C.byref(loss))
        return loss.value

    def loss_tensor(self):
        h = C.c_int64(0)
        self._call("dp_loss_tensor", C.c_int64(self.handle), C.byref(h))
        return Tensor(self.engine, h.value)

    def graph_nodes(self):
        n = C.c_int64(0)
        self._call("dp_graph_nodes", C.c_int64(self.handle), C.byref(n))
        return n.value
