"""Host-side multi-rank logic on CPU ranks (gloo, world size 2): the unique-id hand-off that Comm performs and the
shard arithmetic of the tensor-parallel packing."""
import os
import subprocess
import sys
import textwrap


def test_unique_id_broadcast_and_shard_math_gloo():
    code = textwrap.dedent('''
        import os, sys
        import torch, torch.distributed as dist
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        dist.init_process_group("gloo")
        # the 128-byte id travels as a python object from rank 0, as b200_llama.Comm does
        box = [bytes(range(128)) if rank == 0 else b""]
        dist.broadcast_object_list(box, src=0)
        assert box[0] == bytes(range(128))
        # vocabulary shards of the two ranks tile the vocabulary exactly
        V = 32000
        vl = V // world
        lo = torch.tensor([rank * vl, (rank + 1) * vl])
        allb = [torch.zeros(2, dtype=torch.long) for _ in range(world)]
        dist.all_gather(allb, lo)
        flat = torch.stack(allb).flatten().tolist()
        assert flat[0] == 0 and flat[-1] == V and all(flat[2 * i + 1] == flat[2 * i + 2] for i in range(world - 1))
        # a sum over ranks of per-rank gradients equals the gradient of the summed loss (what allreduce_f32 does)
        g = torch.full((4,), float(rank + 1))
        dist.all_reduce(g)
        assert g.tolist() == [3.0] * 4
        dist.destroy_process_group()
        print("OK", rank)
    ''')
    env = dict(os.environ)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29511", "--no-python", sys.executable, "-c", code],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and r.stdout.count("OK") == 2, r.stdout[-2000:] + r.stderr[-3000:]


def _run_ranks(code, port, timeout=300):
    return subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), "--no-python", sys.executable, "-c",
                           code], capture_output=True, text=True, timeout=timeout, env=dict(os.environ))


PREAMBLE = '''
import os, sys, datetime
sys.path.insert(0, os.path.join(os.getcwd(), "enzyme-jax_b200"))
import torch, torch.distributed as dist
import b200_llama as B
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
'''


def test_id_hand_off_reaches_every_rank_gloo():
    """The hand-off Comm performs (rank 0's id to everybody, then a roll call), with a fake id maker: no GPU, no NCCL."""
    code = PREAMBLE + textwrap.dedent('''
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=30))
        got = B.share_unique_id(rank, world, lambda: bytes(range(128)))
        assert got == bytes(range(128))
        dist.destroy_process_group()
        print("OK", rank)
    ''')
    r = _run_ranks(code, 29512)
    assert r.returncode == 0 and r.stdout.count("OK") == 2, r.stdout[-2000:] + r.stderr[-3000:]


def test_rank_that_leaves_before_the_hand_off_is_detected_on_the_host_gloo():
    """Failure injected on the host: rank 1 exits right after joining, before the id hand-off.  Rank 0 must not hang:
    its hand-off ends with B200Error (NCCL status 8) within the group's timeout, before any GPU work is launched."""
    code = PREAMBLE + textwrap.dedent('''
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=10))
        if rank == 1:
            os._exit(0)  # dies between steps: nothing of it is in flight
        import time
        t0 = time.time()
        try:
            B.share_unique_id(rank, world, lambda: bytes(128))
        except B.B200Error as e:
            assert e.status == 8, e.status
            assert time.time() - t0 < 60
            print("DETECTED", rank)
            os._exit(0)
        print("NOT DETECTED")
        os._exit(3)
    ''')
    r = _run_ranks(code, 29513)
    assert "DETECTED 0" in r.stdout and "NOT DETECTED" not in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
