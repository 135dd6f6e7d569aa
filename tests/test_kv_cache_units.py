"""Dense, sliding-window, per-layer and paged KV caches (crates/nn/src/kv_cache.rs `mod tests`): what is stored, what comes
back, how much memory it takes, and what the 8-bit formats cost in accuracy."""
import pytest
import torch

from rustral_b200.core.errors import InvalidArgument
from rustral_b200.nn import BatchedCache, CacheConfig, CacheQuantization, KVCache, PagedCache, SlidingWindowCache


def _kv(n, seed, heads=2, dim=4, batch=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(batch, heads, n, dim, generator=g), torch.randn(batch, heads, n, dim, generator=g)


def test_dense_cache_appends_in_order_and_refuses_overflow():
    c = KVCache(CacheConfig(num_heads=2, head_dim=4, max_seq_len=8, quantization=CacheQuantization.FP32))
    k1, v1 = _kv(3, 0)
    k2, v2 = _kv(2, 1)
    c.append(k1, v1); c.append(k2, v2)
    k, v = c.get()
    assert c.len == 5 and torch.equal(k, torch.cat([k1, k2], 2)) and torch.equal(v, torch.cat([v1, v2], 2))
    kr, _ = c.get_range(2, 4)
    assert torch.equal(kr, torch.cat([k1, k2], 2)[:, :, 2:4])
    st = c.memory_stats()
    assert st.allocated_bytes == 2 * 2 * 8 * 4 * 4 and st.utilization == 5 / 8 and st.used_bytes == st.allocated_bytes * 5 // 8
    with pytest.raises(InvalidArgument, match="overflow"):
        c.append(*_kv(4, 2))
    c.reset()
    assert c.len == 0 and c.get()[0].shape[2] == 0


def test_cache_config_memory_and_head_sharing():
    cfg = CacheConfig(num_heads=32, head_dim=128, max_seq_len=4096, batch_size=2, num_layers=4)
    assert cfg.num_kv_heads == 32 and cfg.memory_bytes() == 2 * 2 * 32 * 4096 * 128 * 4 * 2      # K and V, bf16
    assert cfg.with_gqa(8).memory_bytes() == 2 * 2 * 8 * 4096 * 128 * 4 * 2
    assert cfg.with_mqa().num_kv_heads == 1
    with pytest.raises(InvalidArgument):
        CacheConfig(num_heads=12, head_dim=64, max_seq_len=16).with_gqa(5)
    assert [q.bytes_per_element for q in CacheQuantization] == [4, 2, 2, 1, 1]


@pytest.mark.parametrize("quant,rel", [(CacheQuantization.BF16, 2 ** -8), (CacheQuantization.FP16, 2 ** -10),
                                       (CacheQuantization.INT8, 1 / 127), (CacheQuantization.FP8, 2 ** -4)])
def test_low_precision_caches_return_values_within_their_format(quant, rel):
    c = KVCache(CacheConfig(num_heads=2, head_dim=4, max_seq_len=16, quantization=quant))
    k, v = _kv(6, 3)
    c.append(k, v)
    kq, vq = c.get()
    assert c.k.element_size() == quant.bytes_per_element
    for got, want in ((kq.float(), k), (vq.float(), v)):
        bound = rel * want.abs().max() if quant is CacheQuantization.INT8 else rel * want.abs() + 2e-3 * want.abs().max()
        assert bool(((got - want).abs() <= bound + 1e-7).all())
    # the scale is fixed by the first append: larger values later saturate instead of corrupting what is stored
    if quant.scaled:
        c.append(10 * k[:, :, :1], 10 * v[:, :, :1])
        k2, _ = c.get()
        assert torch.allclose(k2[:, :, :6].float(), kq.float()) and float(k2[:, :, 6].abs().max()) <= float(k.abs().max()) * 1.01


def test_sliding_window_keeps_the_newest_entries_in_chronological_order():
    cfg = CacheConfig(num_heads=2, head_dim=4, max_seq_len=100, quantization=CacheQuantization.FP32)
    c = SlidingWindowCache(cfg, window=4)
    k, v = _kv(7, 4)
    c.append(k[:, :, :3], v[:, :, :3])
    assert c.len == 3 and torch.equal(c.get()[0], k[:, :, :3])
    c.append(k[:, :, 3:], v[:, :, 3:])
    kw, vw = c.get()
    assert c.len == 4 and c.total == 7 and torch.equal(kw, k[:, :, 3:7]) and torch.equal(vw, v[:, :, 3:7])
    c.reset()
    assert c.len == 0 and c.total == 0
    c.append(k[:, :, :2], v[:, :, :2])
    assert torch.equal(c.get()[0], k[:, :, :2])


def test_quantised_sliding_window_stores_scaled_values_not_truncated_ones():
    cfg = CacheConfig(num_heads=2, head_dim=4, max_seq_len=100, quantization=CacheQuantization.INT8)
    c = SlidingWindowCache(cfg, window=3)
    k, v = _kv(5, 5)
    k, v = 0.3 * k, 0.3 * v                       # all magnitudes below 1: a plain cast to int8 would store zeros
    c.append(k, v)
    kw, vw = c.get()
    assert kw.dtype == torch.float32 and float(kw.abs().max()) > 0.1
    assert torch.allclose(kw, k[:, :, 2:5], atol=float(k.abs().max()) / 127 + 1e-6)
    assert torch.allclose(vw, v[:, :, 2:5], atol=float(v.abs().max()) / 127 + 1e-6)


def test_batched_cache_keeps_layers_apart():
    cfg = CacheConfig(num_heads=2, head_dim=4, max_seq_len=8, quantization=CacheQuantization.FP32)
    c = BatchedCache(3, cfg)
    parts = [_kv(2, 10 + l) for l in range(3)]
    for l, (k, v) in enumerate(parts):
        c.append(l, k, v)
    assert c.len == 2 and all(torch.equal(c.get(l)[0], parts[l][0]) and torch.equal(c.get(l)[1], parts[l][1]) for l in range(3))
    c.reset()
    assert c.len == 0


def test_paged_cache_block_tables_slots_and_reuse():
    c = PagedCache(num_blocks=6, block_size=4, num_layers=1, num_kv_heads=1, head_dim=8)
    assert c.free_blocks == 6 and c.blocks_needed(9) == 3 and c.can_allocate(1, 24) and not c.can_allocate(1, 25)
    assert c.allocate(1, 9) and c.allocate(2, 5)
    t1, t2 = c.block_table(1), c.block_table(2)
    assert len(t1) == 3 and len(t2) == 2 and not set(t1) & set(t2) and c.free_blocks == 1 and c.num_sequences() == 2
    assert c.slot(1, 0) == t1[0] * 4 and c.slot(1, 5) == t1[1] * 4 + 1 and c.slot(1, 8) == t1[2] * 4
    assert not c.allocate(3, 9)                              # two blocks short: refused, nothing changes
    assert c.free_blocks == 1
    assert c.allocate(1, 12) and len(c.block_table(1)) == 3  # growing within the last block needs no new one
    assert c.allocate(1, 13) and len(c.block_table(1)) == 4 and c.free_blocks == 0
    assert c.free(1) == 4 and c.free_blocks == 4 and c.num_sequences() == 1
    assert c.allocate(3, 16) and set(c.block_table(3)) <= set(range(6)) - set(t2)
