"""Host-side logic of the multi-rank path on CPU: the rendezvous that swaps
inbox handles (2 gloo ranks), offset bookkeeping, workload sharding."""
import os
import subprocess
import sys
import textwrap

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_counts_from_inclusive_offsets():
    from apt_b200.exchange import _counts

    assert _counts(torch.tensor([3, 3, 10])) == [3, 0, 7]
    assert _counts(torch.tensor([0])) == [0]


def test_partition_and_batches():
    sys.path.insert(0, ROOT)
    import bench
    from apt_b200 import synthetic

    mv = synthetic.partition_min_vids(103, 4)
    assert mv.tolist() == [0, 25, 50, 75, 103]
    ids = torch.arange(1000)
    bs = bench.batches_of(ids, 64, 40)
    assert all(b.numel() == 64 for b in bs) and bs[0][0] == 0 and bs[1][0] == 64
    w = synthetic.WORKLOADS["c1_papers_np"]
    assert w.scale == 27 and w.fanouts == [15, 10, 5] and w.batch == 1024


def test_handle_exchange_two_gloo_ranks(tmp_path):
    """exchange_blobs is what carries the 64-byte IPC handles between ranks."""
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {ROOT!r})
        import torch.distributed as dist
        from apt_b200.exchange import exchange_blobs, make_exchange
        from apt_b200.ops import NPCState
        dist.init_process_group("gloo")
        r = dist.get_rank()
        blobs = exchange_blobs(bytes([r]) * 64)
        assert blobs == [bytes([0]) * 64, bytes([1]) * 64], blobs
        s = NPCState(); s.world_size = 1
        assert make_exchange(s).name == "local"
        s.world_size = 2; s.shuffle_backend = "bogus"
        try:
            make_exchange(s)
        except RuntimeError as e:
            assert "unknown" in str(e)
        else:
            raise SystemExit("bad backend accepted")
        dist.barrier()
        print("HOST_OK", r)
    """))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29431", str(script)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, MASTER_ADDR="127.0.0.1"))
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert res.stdout.count("HOST_OK") == 2
