"""Attention modules against plain tensor math (crates/nn/src/attention.rs `mod tests`): head sharing, masks of both
kinds, rotary offsets, the memory estimate and the feed-forward blocks."""
import math

import pytest
import torch

from rustral_b200.core import CpuBackend, ForwardCtx
from rustral_b200.core.errors import InvalidArgument
from rustral_b200.nn import (AttentionMemoryStats, FlashAttention, FlashAttentionConfig, MultiHeadAttention, SelfAttention,
                             SelfAttentionConfig, SwiGLUFeedForward, TapeFeedForward, causal_mask, scaled_dot_product_attention)
from rustral_b200.nn.attention import KeyPaddingMask

BE = CpuBackend()
CTX = ForwardCtx.inference(BE)


def _ref_attention(q, k, v, causal=False, lens=None):
    """[B,S,H,D] inputs; explicit softmax(QK^T / sqrt(D)) V with optional causal and key-length masking."""
    B, S, H, D = q.shape
    rep = H // k.shape[2]
    qh, kh, vh = q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3).repeat_interleave(rep, 1), v.permute(0, 2, 1, 3).repeat_interleave(rep, 1)
    s = qh @ kh.transpose(-1, -2) / math.sqrt(D)
    Sk = k.shape[1]
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(S, Sk, dtype=torch.bool), 1 + Sk - S), float("-inf"))
    if lens is not None:
        hide = torch.arange(Sk)[None, :] >= torch.as_tensor(lens)[:, None]
        s = s.masked_fill(hide[:, None, None, :], float("-inf"))
    return (torch.softmax(s, -1) @ vh).permute(0, 2, 1, 3)


def _qkv(B=2, S=6, H=4, Hkv=4, D=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, S, H, D, generator=g), torch.randn(B, S, Hkv, D, generator=g), torch.randn(B, S, Hkv, D, generator=g))


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("hkv", [4, 2, 1])
def test_attention_function_matches_explicit_softmax_for_mha_gqa_and_mqa(causal, hkv):
    q, k, v = _qkv(Hkv=hkv)
    assert torch.allclose(scaled_dot_product_attention(q, k, v, None, causal), _ref_attention(q, k, v, causal), atol=1e-5)


def test_key_padding_lengths_and_an_additive_mask_tensor_agree():
    q, k, v = _qkv(seed=1)
    lens = [6, 3]
    by_len = scaled_dot_product_attention(q, k, v, KeyPaddingMask(lens))
    add = torch.zeros(2, 1, 1, 6)
    add[1, :, :, 3:] = float("-inf")
    by_tensor = scaled_dot_product_attention(q, k, v, add)
    assert torch.allclose(by_len, by_tensor, atol=1e-5) and torch.allclose(by_len, _ref_attention(q, k, v, lens=lens), atol=1e-5)
    ids = torch.tensor([[5, 6, 7, 8, 9, 4], [3, 3, 9, 0, 0, 0]])
    assert KeyPaddingMask.from_token_ids(ids, pad_id=0).lengths.tolist() == [6, 3]


def test_causal_module_stays_causal_when_given_key_padding_lengths():
    att = SelfAttention.new(BE, SelfAttentionConfig(16, 4, causal=True), seed=2, scale=0.3)
    x = torch.randn(2, 6, 16, generator=torch.Generator().manual_seed(3))
    y = att(x, CTX, KeyPaddingMask([6, 4]))
    x2 = x.clone()
    x2[:, 3] += 1.0                                            # a later token must not change earlier outputs
    y2 = att(x2, CTX, KeyPaddingMask([6, 4]))
    assert torch.allclose(y[:, :3], y2[:, :3], atol=1e-6) and not torch.allclose(y[:, 3:], y2[:, 3:], atol=1e-4)
    x3 = x.clone()
    x3[1, 5] += 5.0                                            # a padded key of row 1 must not change that row's real positions
    y3 = att(x3, CTX, KeyPaddingMask([6, 4]))
    assert torch.allclose(y[1, :4], y3[1, :4], atol=1e-6)
    # an additive tensor replaces the module's own causal mask: the caller supplies the whole mask
    full = att(x, CTX, causal_mask(BE, 6))
    assert torch.allclose(full, att(x, CTX), atol=1e-5)


def test_self_attention_equals_projections_plus_reference_attention_and_takes_rank_2_input():
    cfg = SelfAttentionConfig(16, 4, num_kv_heads=2)
    att = SelfAttention.new(BE, cfg, seed=4, scale=0.3)
    x = torch.randn(2, 5, 16, generator=torch.Generator().manual_seed(5))
    q, k, v, o = (p for p in att._proj)
    qh = (x @ q.weight.tensor.t() + q.bias.tensor).reshape(2, 5, 4, 4)
    kh = (x @ k.weight.tensor.t() + k.bias.tensor).reshape(2, 5, 2, 4)
    vh = (x @ v.weight.tensor.t() + v.bias.tensor).reshape(2, 5, 2, 4)
    want = _ref_attention(qh, kh, vh).reshape(2, 5, 16) @ o.weight.tensor.t() + o.bias.tensor
    assert torch.allclose(att(x, CTX), want, atol=1e-5)
    assert torch.allclose(att(x[0], CTX), want[0], atol=1e-5)              # [S, d] is batch 1
    res = torch.randn(2, 5, 16, generator=torch.Generator().manual_seed(6))
    assert torch.allclose(att(x, CTX, None, res), want + res, atol=1e-5)  # the residual rides in the output projection
    assert [n for n, _ in att.named_parameters()][:2] == ["q_proj.weight", "q_proj.bias"]
    assert att._proj[1].weight.tensor.shape == (8, 16)                    # two KV heads of 4
    with pytest.raises(InvalidArgument):
        SelfAttentionConfig(16, 3)
    with pytest.raises(InvalidArgument):
        SelfAttentionConfig(16, 4, num_kv_heads=3)


def test_rotary_attention_with_an_offset_continues_a_sequence():
    """The last position of a full causal pass equals a one-token pass at pos_offset = S - 1 over the same keys only when
    the rotation depends on absolute positions: shifting the whole window changes nothing but the offset."""
    att = SelfAttention.new(BE, SelfAttentionConfig(16, 2, causal=True, rope_theta=10000.0, bias=False), seed=7, scale=0.3)
    x = torch.randn(1, 6, 16, generator=torch.Generator().manual_seed(8))
    a = att(x, CTX)
    b = att(x, CTX, pos_offset=11)
    assert torch.allclose(a, b, atol=1e-5)                    # scores depend on position differences only
    plain = SelfAttention.new(BE, SelfAttentionConfig(16, 2, causal=True, bias=False), seed=7, scale=0.3)
    assert not torch.allclose(a, plain(x, CTX), atol=1e-4)   # and the rotation really is applied
    assert len(att.parameters()) == 4                         # bias=False


def test_flash_attention_and_multi_head_wrappers_are_the_same_computation():
    fa = FlashAttention.new(BE, FlashAttentionConfig(16, 4, causal=True), seed=9)
    sa = SelfAttention.new(BE, SelfAttentionConfig(16, 4, causal=True), seed=9)
    x = torch.randn(2, 7, 16, generator=torch.Generator().manual_seed(10))
    assert torch.equal(fa(x, CTX), sa(x, CTX)) and fa.flash_config.block_size == 128
    mha = MultiHeadAttention.new(BE, 16, 4, seed=9)
    assert [n for n, _ in mha.named_parameters()][0] == "attention.q_proj.weight"
    assert mha(x, CTX).shape == x.shape


def test_attention_memory_estimate():
    st = AttentionMemoryStats.calculate(batch=4, seq=4096, heads=32, head_dim=128, block_size=128, elem_bytes=2)
    qkv = 3 * 4 * 4096 * 32 * 128 * 2
    assert st.standard_bytes == qkv + 4 * 32 * 4096 * 4096 * 2 * 2
    assert st.flash_bytes == qkv + 4 * 32 * 4096 * 4 + 32 * 128 * 128 * 4
    assert st.savings_ratio == pytest.approx(st.standard_bytes / st.flash_bytes) and st.savings_ratio > 20
    short = AttentionMemoryStats.calculate(1, 128, 4, 64)
    assert short.savings_ratio < st.savings_ratio            # the saving grows with the sequence length


def test_feed_forward_blocks_match_their_formulas_with_and_without_bias():
    x = torch.randn(3, 5, 16, generator=torch.Generator().manual_seed(11))
    gelu = lambda t: torch.nn.functional.gelu(t, approximate="tanh")
    for bias in (True, False):
        ff = TapeFeedForward.new(BE, 16, 32, seed=12, bias=bias, scale=0.3)
        h = x @ ff.fc1.weight.tensor.t() + (ff.fc1.bias.tensor if bias else 0)
        want = gelu(h) @ ff.fc2.weight.tensor.t() + (ff.fc2.bias.tensor if bias else 0)
        assert torch.allclose(ff(x, CTX), want, atol=1e-5)
        assert torch.allclose(ff(x, CTX, x), want + x, atol=1e-5)
        xg = x.clone().requires_grad_()
        ff(xg, ForwardCtx.train(BE)).sum().backward()
        assert xg.grad is not None and all(p.tensor.grad is not None for p in ff.parameters())
        ff.zero_grad()
    sw = SwiGLUFeedForward.new(BE, 16, 24, seed=13, scale=0.3)
    gu = x @ sw.gate_up.weight.tensor.t()
    want = (torch.nn.functional.silu(gu[..., :24]) * gu[..., 24:]) @ sw.down.weight.tensor.t()
    assert torch.allclose(sw(x, CTX), want, atol=1e-5)


def test_key_padding_lengths_from_an_additive_mask_tensor():
    q, k, v = _qkv(seed=21)
    add = torch.zeros(2, 1, 1, 6)
    add[1, :, :, 4:] = float("-inf")
    kp = KeyPaddingMask.from_additive(add)
    assert kp.lengths.tolist() == [6, 4]
    assert torch.allclose(scaled_dot_product_attention(q, k, v, kp), scaled_dot_product_attention(q, k, v, add), atol=1e-5)
    assert KeyPaddingMask.from_additive(torch.tensor([[0.0, -1e9, -1e9], [0.0, 0.0, 0.0]])).lengths.tolist() == [1, 3]
    holes = torch.tensor([[0.0, float("-inf"), 0.0]])                      # padding in the middle is not a length
    assert KeyPaddingMask.from_additive(holes) is None and KeyPaddingMask.from_additive(holes, check=False).lengths.tolist() == [2]
    assert KeyPaddingMask.from_additive(torch.zeros(2, 4, 6, 6)) is None   # a full [B, H, S, S] mask is not a key mask
