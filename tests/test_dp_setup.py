"""Host-side failures of a data-parallel job, on CPU ranks (gloo): a rank that never joins, ranks that disagree on the
flat gradient length.  Nothing here touches a GPU: the failure is made on the host and must surface as an exception on
every rank that is still there."""
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_WORKER = r"""
import os, sys, time
sys.path.insert(0, os.environ["RT_ROOT"])
from rusttensor_b200 import dp_setup
rank, world, case = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), os.environ["CASE"]
t0 = time.time()
try:
    dist = dp_setup.rendezvous("gloo", rank, world, port=int(os.environ["RT_PORT"]), timeout_s=float(os.environ.get("RT_TIMEOUT", "30")))
except dp_setup.RendezvousError as e:
    print("RENDEZVOUS_ERROR %.1f %s" % (time.time() - t0, e)); sys.exit(3)
if case == "mismatch":
    flat_len = 421642 if rank == 0 else 421646          # as if rank 1 had been started with another model
    try:
        dp_setup.agree(dist, "the flat gradient length", [flat_len, 8])
    except dp_setup.LayoutMismatch as e:
        print("MISMATCH", e); dist.destroy_process_group(); sys.exit(4)
elif case == "count_mismatch":
    try:
        dp_setup.agree(dist, "the parameter list", [1, 2, 3][: 2 + rank])
    except dp_setup.LayoutMismatch as e:
        print("MISMATCH", e); dist.destroy_process_group(); sys.exit(4)
else:
    got = dp_setup.agree(dist, "the flat gradient length", [421642, 8])
    ident = dp_setup.share_unique_id(dist, lambda: bytes(range(128)), rank)
    assert got == [421642, 8] and ident == list(range(128))
    print("AGREED")
dist.destroy_process_group()
"""


def _run(tmp_path, case, ranks, world=2, timeout_s="30"):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    port = str(31500 + (os.getpid() * 7 + hash(case)) % 2000)
    procs = []
    for rank in ranks:
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), RT_ROOT=ROOT, RT_PORT=port, CASE=case, RT_TIMEOUT=timeout_s)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=240) for p in procs]
    return [(p.returncode, o[0], o[1]) for p, o in zip(procs, outs)]


def test_a_rank_that_never_joins_ends_the_rendezvous_with_an_error(tmp_path):
    t0 = time.time()
    (rc, out, err), = _run(tmp_path, "ok", ranks=[0], timeout_s="4")
    assert rc == 3 and "RENDEZVOUS_ERROR" in out, (rc, out, err[-2000:])
    assert "did not join within 4 s" in out
    assert time.time() - t0 < 120


def test_ranks_that_disagree_on_the_flat_length_all_raise(tmp_path):
    res = _run(tmp_path, "mismatch", ranks=[0, 1])
    for rc, out, err in res:
        assert rc == 4 and "MISMATCH" in out, (rc, out, err[-2000:])
        assert "rank 0: [421642, 8]" in out and "rank 1: [421646, 8]" in out


def test_ranks_that_pass_different_numbers_of_values_all_raise(tmp_path):
    res = _run(tmp_path, "count_mismatch", ranks=[0, 1])
    for rc, out, err in res:
        assert rc == 4 and "rank 0: 2 values" in out and "rank 1: 3 values" in out, (rc, out, err[-2000:])


def test_matching_ranks_agree_and_share_the_communicator_id(tmp_path):
    res = _run(tmp_path, "ok", ranks=[0, 1])
    for rc, out, err in res:
        assert rc == 0 and "AGREED" in out, (rc, out, err[-2000:])
