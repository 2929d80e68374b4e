"""KV pack / unpack / transfer kernels: bit-exact against torch index copies."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(prompt_lens, page=64, row=256, blocks=None):
    from dlslime_b200.ops import kv

    pages = sum((n + page - 1) // page for n in prompt_lens)
    blocks = blocks or pages + 7
    g = torch.Generator().manual_seed(3)
    dst_blocks = torch.randperm(blocks, generator=g)[:pages].tolist()
    tasks = kv.build_page_tasks(prompt_lens, page, dst_blocks)
    return tasks, dst_blocks, blocks


def test_pack_unpack_roundtrip_bit_exact():
    from dlslime_b200.ops import kv
    from dlslime_b200.ops._common import default_status

    lens, page, row = [100, 64, 1, 513, 129], 64, 256
    (tok_off, blk, ntok), dst_blocks, blocks = _setup(lens, page, row)
    total = sum(lens)
    src = torch.randn(2, total, row, device="cuda").to(torch.bfloat16)
    paged = torch.zeros(2, blocks, page, row, device="cuda", dtype=torch.bfloat16)
    kv.kv_pack(src, paged, tok_off, blk, ntok)
    torch.cuda.synchronize()
    default_status().check()
    expect = torch.zeros_like(paged)
    for t, b, n in zip(tok_off.tolist(), blk.tolist(), ntok.tolist()):
        expect[:, b, :n] = src[:, t:t + n]
    assert torch.equal(paged, expect)
    back = torch.zeros_like(src)
    kv.kv_unpack(paged, back, tok_off, blk, ntok)
    torch.cuda.synchronize()
    assert torch.equal(back, src)


def test_out_of_range_block_is_reported_not_written():
    from dlslime_b200.ops import kv
    from dlslime_b200.ops._common import default_status

    page, row = 64, 256
    src = torch.randn(2, 128, row, device="cuda").to(torch.bfloat16)
    paged = torch.zeros(2, 4, page, row, device="cuda", dtype=torch.bfloat16)
    tok_off = torch.tensor([0, 64], dtype=torch.int32, device="cuda")
    blk = torch.tensor([1, 9], dtype=torch.int32, device="cuda")  # block 9 does not exist
    kv.kv_pack(src, paged, tok_off, blk)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError):
        default_status().check()
    assert torch.equal(paged[:, 1], src[:, :64]) and paged[:, [0, 2, 3]].abs().sum() == 0


def test_prefill_sender_pushes_every_layer_with_flags():
    """Emulated peer on one GPU: the 'decode' cache is a second region on the same device."""
    from dlslime_b200.models.pd_kv import KVShape, PagedKVCache, PrefillSender, wait_layers
    from dlslime_b200.ops._common import default_status
    from dlslime_b200.parallel.symm import SymmetricHeap

    shape = KVShape(layers=4, kv_heads_local=2, head_dim=128, page_tokens=64)
    lens = [130, 64, 700]
    pages = sum((n + 63) // 64 for n in lens)
    blocks = pages + 5
    heap = SymmetricHeap.emulated(2, PagedKVCache.bytes_needed(shape, blocks))
    cache = PagedKVCache(shape, blocks, heap, owner_rank=1)
    sender = PrefillSender(shape, cache, max_tokens=sum(lens), comm_blocks=16)
    g = torch.Generator().manual_seed(5)
    dst_blocks = torch.randperm(blocks, generator=g)[:pages].tolist()
    tok_off, blk, ntok = sender.plan(lens, dst_blocks)
    sender.kv_stage.copy_(torch.randn(sender.kv_stage.shape, device="cuda"))
    d = 256
    hidden = torch.randn(sum(lens), d, device="cuda").to(torch.bfloat16)
    weights = [(torch.randn(d, d, device="cuda") * 0.05).to(torch.bfloat16)]
    sender.run_prefill_with_transfer(hidden, weights, overlap=True)
    torch.cuda.synchronize()
    default_status().check()
    assert wait_layers(cache, sender.step, timeout_s=2.0)
    got = cache.tensor()
    for t, b, n in zip(tok_off.tolist(), blk.tolist(), ntok.tolist()):
        assert torch.equal(got[:, :, b, :n], sender.kv_stage[:, :, t:t + n])
