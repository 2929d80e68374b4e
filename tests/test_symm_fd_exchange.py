"""Host side of the multicast heap: the file-descriptor exchange between ranks (Unix sockets, SCM_RIGHTS), run as
three gloo ranks on the CPU. Every rank sends a pipe's read end (rank 0 two descriptors, as it does with the multicast
object), and the receivers read through what they got."""
import os
import subprocess
import sys
import textwrap

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_descriptors_travel_between_ranks(tmp_path):
    body = textwrap.dedent(f"""
        import os, sys, torch.distributed as dist
        sys.path.insert(0, {REPO!r})
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        from dlslime_b200.parallel.symm import SymmetricHeap
        h = SymmetricHeap.__new__(SymmetricHeap)          # only the exchange is under test: no device memory
        h.world, h.rank, h.group = world, rank, None
        r, w = os.pipe()
        os.write(w, f"hello from {{rank}}".encode())
        got = h._exchange_fds("cputest", [r] + ([w] if rank == 0 else []))
        assert sorted(got) == [p for p in range(world) if p != rank]
        for src, fds in got.items():
            assert len(fds) == (2 if src == 0 else 1), (src, fds)
        src = (rank - 1) % world                          # each message is read by exactly one receiver
        assert os.read(got[src][0], 100).decode() == f"hello from {{src}}"
        assert h._all_agree(True) and not h._all_agree(rank != 1)
        dist.barrier()
        print("ok", rank)
    """)
    script = tmp_path / "fdx.py"
    script.write_text(body)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "3", "--master-addr", "127.0.0.1",
                        "--master-port", "29656", str(script)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.count("ok") == 3, r.stdout[-2000:] + r.stderr[-3000:]
