"""Low-latency all-to-all on one GPU: every rank of an emulated group issues its stores, then every rank waits."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _exchange(group, xs, **kw):
    hooks = [g.all_to_all_ll_hook(x, **kw_r) for g, x, kw_r in zip(group, xs, _per_rank(kw, len(group)))]
    outs = [h() for h in hooks]
    torch.cuda.synchronize()
    group[0].status.check()
    return outs


def _per_rank(kw, world):
    return [{k: (v[r] if isinstance(v, list) else v) for k, v in kw.items()} for r in range(world)]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_uniform_and_transposed(world):
    from dlslime_b200.ops.alltoall import AllToAllLLBuffer

    msg = 1024 + 8  # rows that do not fill a whole 512-byte piece at the end
    group = AllToAllLLBuffer.emulated_group(world, 32, msg, torch.bfloat16)
    gen = torch.Generator(device="cuda").manual_seed(world)
    for bs in [1, 5, 32, 5]:  # both halves of the double buffer are reused
        xs = [torch.randn((world * bs, msg), generator=gen, device="cuda").to(torch.bfloat16) for _ in range(world)]
        outs = _exchange(group, xs)
        for r in range(world):
            ref = torch.cat([xs[s][r * bs:(r + 1) * bs] for s in range(world)], dim=0)
            assert torch.equal(outs[r], ref), f"rank {r} bs={bs}"
        outs = _exchange(group, xs, is_transpose=True)
        for r in range(world):
            ref = torch.stack([xs[s][r * bs:(r + 1) * bs] for s in range(world)], dim=1)  # [bs, world, msg]
            assert outs[r].shape == (bs, world, msg)
            assert torch.equal(outs[r], ref), f"rank {r} bs={bs} transposed"


def test_variable_split_and_mask():
    from dlslime_b200.ops.alltoall import AllToAllLLBuffer

    world, msg, cap = 4, 512, 16
    group = AllToAllLLBuffer.emulated_group(world, cap, msg, torch.float16)
    gen = torch.Generator(device="cuda").manual_seed(9)
    splits = [[3, 0, 16, 1], [0, 0, 0, 0], [16, 16, 16, 16], [1, 2, 3, 4]]  # splits[s][p]: rows rank s sends to rank p
    xs, offs = [], []
    for s in range(world):
        o = [0]
        for n in splits[s]:
            o.append(o[-1] + n)
        offs.append(torch.tensor(o, dtype=torch.int32, device="cuda"))
        xs.append(torch.randn((max(o[-1], 1), msg), generator=gen, device="cuda").to(torch.float16)[:o[-1]].contiguous())
    masks = [torch.tensor([1, 1, 0, 1], dtype=torch.int32, device="cuda") if s == 3 else None for s in range(world)]
    for _ in range(3):
        outs = _exchange(group, xs, offsets=offs, mask=masks)
        for r in range(world):
            data, counts = outs[r]
            assert data.shape == (world, cap, msg)
            for s in range(world):
                n = splits[s][r] if not (s == 3 and r == 2) else 0  # rank 3 masks destination 2 out
                assert int(counts[s]) == n, (r, s, counts)
                begin = sum(splits[s][:r])
                assert torch.equal(data[s, :n], xs[s][begin:begin + n])


def test_bad_requests_are_refused():
    from dlslime_b200.ops.alltoall import AllToAllIntraLLBuffer
    from dlslime_b200.ops._common import default_status

    g = AllToAllIntraLLBuffer.emulated_group(2, 4, 256, torch.bfloat16)[0]
    with pytest.raises(ValueError):
        g.all_to_all_ll_hook(torch.zeros((3, 256), dtype=torch.bfloat16, device="cuda"))  # not a multiple of world
    with pytest.raises(ValueError):
        g.all_to_all_ll_hook(torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda"))  # 8 rows per rank > max_bs
    with pytest.raises(ValueError):
        g.set_max_bs(5)
    assert AllToAllIntraLLBuffer.get_buffer_size_hint(4, 256, torch.bfloat16, 2) == 2 * 2 * 2048 + 4096
    # a split that exceeds the slot is caught on the device: reported, nothing is stored for that destination
    off = torch.tensor([0, 6, 6], dtype=torch.int32, device="cuda")
    g.all_to_all_ll_hook(torch.ones((6, 256), dtype=torch.bfloat16, device="cuda"), offsets=off)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError):
        default_status().check()
