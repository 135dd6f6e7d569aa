"""The hand-scheduled backward of the fused engine against torch.autograd on the same parameters (CPU, fp32)."""
import math

import pytest
import torch

from rustral_b200.models.config import preset
from rustral_b200.runtime.fused_gpt import FusedGPTEngine


def _gelu(x):
    return 0.5 * x * (1 + torch.tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * x ** 3)))


def _rope(x, theta):
    B, S, H, D = x.shape
    half = D // 2
    inv = theta ** (-2.0 * torch.arange(half, dtype=torch.float32) / D)
    ang = torch.arange(S, dtype=torch.float32)[:, None] * inv[None]
    c, s = torch.cos(ang)[None, :, None, :], torch.sin(ang)[None, :, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x1 * c + x0 * s], -1)


def reference_loss(cfg, W, ids, targets):
    """Plain torch forward of the same architecture; W maps flat-engine names to leaf tensors."""
    B, S = ids.shape
    d, H, Hk, D = cfg.d_model, cfg.n_head, cfg.n_kv_head, cfg.head_dim
    rms = cfg.arch == "llama"

    def norm(x, p):
        if rms:
            return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + cfg.norm_eps) * W[p + ".weight"]
        mu = x.mean(-1, keepdim=True)
        var = ((x - mu) ** 2).mean(-1, keepdim=True)
        return (x - mu) * torch.rsqrt(var + cfg.norm_eps) * W[p + ".weight"] + W[p + ".bias"]

    x = W["tok_embed.embed"][ids]
    if not rms:
        x = x + W["pos_embed.embed"][torch.arange(S)][None]
    for l in range(cfg.n_layer):
        p = f"layers.{l}."
        h = norm(x, p + "ln1")
        qkv = h @ W[p + "attn.wqkv.weight"].t()
        if not rms:
            qkv = qkv + W[p + "attn.wqkv.bias"]
        q = qkv[..., :H * D].reshape(B, S, H, D)
        k = qkv[..., H * D:(H + Hk) * D].reshape(B, S, Hk, D)
        v = qkv[..., (H + Hk) * D:].reshape(B, S, Hk, D)
        if rms:
            q, k = _rope(q, cfg.rope_theta), _rope(k, cfg.rope_theta)
        qh = q.permute(0, 2, 1, 3)
        kh = k.permute(0, 2, 1, 3).repeat_interleave(H // Hk, 1)
        vh = v.permute(0, 2, 1, 3).repeat_interleave(H // Hk, 1)
        s = qh @ kh.transpose(-1, -2) / math.sqrt(D)
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
        a = (torch.softmax(s, -1) @ vh).permute(0, 2, 1, 3).reshape(B, S, d)
        a = a @ W[p + "attn.wo.weight"].t()
        if not rms:
            a = a + W[p + "attn.wo.bias"]
        x = x + a
        h = norm(x, p + "ln2")
        if rms:
            gu = h @ W[p + "ffn.gate_up.weight"].t()
            f = cfg.ffn_dim
            m = (torch.nn.functional.silu(gu[..., :f]) * gu[..., f:]) @ W[p + "ffn.down.weight"].t()
        else:
            m = _gelu(h @ W[p + "ffn.fc1.weight"].t() + W[p + "ffn.fc1.bias"]) @ W[p + "ffn.fc2.weight"].t() + W[p + "ffn.fc2.bias"]
        x = x + m
    x = norm(x, "final_norm")
    head = W["tok_embed.embed" if cfg.tie_embeddings else "head.weight"]
    logits = (x @ head.t())[..., :cfg.vocab_size]
    return torch.nn.functional.cross_entropy(logits.reshape(-1, cfg.vocab_size), targets.reshape(-1))


@pytest.mark.parametrize("name", ["gpt2-test", "llama-test"])
def test_engine_gradients_match_autograd(name):
    cfg = preset(name, seq_len=16, d_model=64, ffn_dim=128, vocab_size=96, vocab_multiple=32)
    eng = FusedGPTEngine(cfg, "cpu", micro_batch=2, seed=3)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len), generator=g)
    tg = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len), generator=g)
    loss = eng.train_step(ids, tg, do_step=False)            # two micro-batches: exercises accumulation
    W = {s.name: eng.params.view(eng.params.master, s.name).clone().requires_grad_() for s in eng.params.specs}
    ref = reference_loss(cfg, W, ids, tg)
    ref.backward()
    assert abs(float(loss) - float(ref)) < 1e-4
    for s in eng.params.specs:
        got, want = eng.params.g(s.name), W[s.name].grad
        assert want is not None, s.name
        err = (got - want).abs().max().item()
        assert err <= 1e-4 * (want.abs().max().item() + 1e-3) + 1e-6, f"{s.name}: {err}"


def test_engine_state_dict_roundtrip_is_strict():
    from rustral_b200.core.errors import SerializationError, ShapeMismatch
    cfg = preset("gpt2-test", seq_len=16, d_model=64, ffn_dim=128, vocab_size=96, vocab_multiple=32)
    a, b = FusedGPTEngine(cfg, "cpu", seed=1), FusedGPTEngine(cfg, "cpu", seed=2)
    sd = a.params.state_dict()
    assert "layers.0.attn.wq.weight" in sd and sd["tok_embed.embed"].shape == (96, 64)
    b.params.load_state_dict(sd)
    ids = torch.randint(0, 96, (2, 16))
    assert torch.equal(a.logits(ids), b.logits(ids))
    bad = dict(sd)
    bad.pop("final_norm.weight")
    with pytest.raises(SerializationError):
        b.params.load_state_dict(bad)
    bad = dict(sd)
    bad["extra"] = torch.zeros(1)
    with pytest.raises(SerializationError):
        b.params.load_state_dict(bad)
    bad = dict(sd)
    bad["final_norm.weight"] = torch.zeros(3)
    with pytest.raises(ShapeMismatch):
        b.params.load_state_dict(bad)


def test_hugging_face_checkpoints_convert_and_reproduce_hf_logits():
    """Independent oracle: random GPT-2 and Llama (GQA, rotary) models built by the `transformers` library, converted
    with utils.hf, give the same logits through this framework's engine (CPU, fp32) to round-off."""
    transformers = pytest.importorskip("transformers")
    from rustral_b200.runtime.fused_gpt import FusedGPTEngine
    from rustral_b200.utils.hf import config_from_hf, convert_hf_gpt2, convert_hf_llama
    torch.manual_seed(0)
    ids = torch.randint(0, 300, (2, 32))
    hc = transformers.GPT2Config(vocab_size=300, n_positions=32, n_embd=64, n_layer=2, n_head=4, resid_pdrop=0.0,
                                 embd_pdrop=0.0, attn_pdrop=0.0)
    lc = transformers.LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32, rope_theta=10000.0,
                                  rms_norm_eps=1e-5, tie_word_embeddings=False, attention_dropout=0.0)
    for hf_cfg, cls, conv in ((hc, transformers.GPT2LMHeadModel, convert_hf_gpt2), (lc, transformers.LlamaForCausalLM, convert_hf_llama)):
        model = cls(hf_cfg).eval()
        cfg = config_from_hf(hf_cfg)
        eng = FusedGPTEngine(cfg, "cpu")
        eng.params.load_state_dict(conv(model.state_dict()))            # strict: every name and shape must line up
        with torch.no_grad():
            ref = model(ids).logits
        out = eng.logits(ids)[..., :300]
        assert (out - ref).abs().max().item() < 1e-5, cfg.arch
        # the hand-scheduled backward pass against Hugging Face's autograd: loss and a gradient of every kind
        tgt = torch.randint(0, 300, (2, 32), generator=torch.Generator().manual_seed(3))
        eng2 = FusedGPTEngine(cfg, "cpu", micro_batch=2)
        eng2.params.load_state_dict(conv(model.state_dict()))
        loss = eng2.train_step(ids, tgt, do_step=False)
        model.zero_grad()
        hf_loss = torch.nn.functional.cross_entropy(model(ids).logits.reshape(-1, 300), tgt.reshape(-1))
        hf_loss.backward()
        assert abs(float(loss) - float(hf_loss.detach())) < 1e-5
        hf_grads = {k: v.grad for k, v in model.named_parameters()}
        if cfg.arch == "gpt2":
            pairs = [("layers.1.ffn.fc1.weight", hf_grads["transformer.h.1.mlp.c_fc.weight"].t()),
                     ("layers.0.attn.wo.weight", hf_grads["transformer.h.0.attn.c_proj.weight"].t()),
                     ("layers.0.ln1.bias", hf_grads["transformer.h.0.ln_1.bias"]),
                     ("pos_embed.embed", hf_grads["transformer.wpe.weight"]),
                     ("tok_embed.embed", hf_grads["transformer.wte.weight"])]          # tied: embedding + LM head
        else:
            pairs = [("layers.1.ffn.down.weight", hf_grads["model.layers.1.mlp.down_proj.weight"]),
                     ("layers.0.attn.wo.weight", hf_grads["model.layers.0.self_attn.o_proj.weight"]),
                     ("layers.0.ln1.weight", hf_grads["model.layers.0.input_layernorm.weight"]),
                     ("head.weight", hf_grads["lm_head.weight"]),
                     ("tok_embed.embed", hf_grads["model.embed_tokens.weight"])]
        for name, want in pairs:
            got = eng2.params.g(name)[:want.shape[0]]
            err = (got - want).abs().max().item()
            assert err <= 1e-4 * (want.abs().max().item() + 1e-3) + 1e-6, f"{cfg.arch} {name}: {err}"
    assert config_from_hf(lc).n_kv_head == 2 and config_from_hf(hc).tie_embeddings
    with pytest.raises(ValueError):
        config_from_hf({"model_type": "bert"})


def test_trainer_fits_a_token_file_through_the_native_prefetcher(tmp_path):
    """End to end on the CPU backend: token file -> C++ prefetcher -> LMTrainer; the loss falls on a periodic corpus,
    and a run resumed at step k sees the data an uninterrupted run saw."""
    import numpy as np
    from rustral_b200.data.datasets import TokenFileDataset
    from rustral_b200.runtime.lm_trainer import LMTrainer, TrainConfig
    cfg = preset("gpt2-test", seq_len=16, d_model=32, ffn_dim=64, n_layer=1, n_head=2, vocab_size=64)
    path = tmp_path / "corpus.bin"
    (np.arange(20000) % 11).astype(np.uint16).tofile(path)                 # period-11 sequence: easy to predict
    seen = []
    tr = LMTrainer(cfg, TrainConfig(global_batch=8, micro_batch=8, lr=3e-3, weight_decay=0.0, seed=0), "cpu")
    ds = TokenFileDataset(str(path), seq_len=16, seed=3)
    losses = tr.fit_token_file(ds, 30, on_step=lambda s, l: seen.append(s), lr_schedule=lambda s: 3e-3)
    assert seen == list(range(30)) and losses[-1] < 0.5 * losses[0], (losses[0], losses[-1])
    a = LMTrainer(cfg, TrainConfig(global_batch=8, micro_batch=8, lr=1e-3, seed=1), "cpu")
    b = LMTrainer(cfg, TrainConfig(global_batch=8, micro_batch=8, lr=1e-3, seed=1), "cpu")
    la = a.fit_token_file(ds, 6)
    lb = b.fit_token_file(ds, 3) + b.fit_token_file(ds, 3, first_step=3)
    assert la == lb                                                         # same data, bit-identical trajectory
    with pytest.raises(ValueError):
        tr.fit_token_file(TokenFileDataset(str(path), seq_len=8), 1)


def test_resume_with_optimizer_state_continues_bit_for_bit():
    """Weights + Adam moments + step count: a run stopped after 3 steps and resumed in a fresh trainer reproduces the
    uninterrupted 6-step run exactly; without the optimizer state it does not."""
    from rustral_b200.core.errors import SerializationError
    from rustral_b200.runtime.lm_trainer import LMTrainer, TrainConfig
    cfg = preset("llama-test", seq_len=16, d_model=32, ffn_dim=64, n_layer=1, n_head=2, n_kv_head=1, vocab_size=64)
    tc = lambda: TrainConfig(global_batch=4, micro_batch=4, lr=1e-2, seed=0)
    g = torch.Generator().manual_seed(0)
    batches = [torch.randint(0, 64, (4, 17), generator=g) for _ in range(6)]
    full = LMTrainer(cfg, tc(), "cpu")
    want = [full.step(b) for b in batches]
    first = LMTrainer(cfg, tc(), "cpu")
    got = [first.step(b) for b in batches[:3]]
    weights, (opt_tensors, opt_meta) = first.state_dict(), first.optimizer_state()
    assert opt_meta["step"] == 3 and opt_tensors["adam.m"].abs().sum() > 0
    resumed = LMTrainer(cfg, tc(), "cpu")
    resumed.load_state_dict(weights)
    resumed.load_optimizer_state(opt_tensors, opt_meta)
    got += [resumed.step(b) for b in batches[3:]]
    assert got == want
    cold = LMTrainer(cfg, tc(), "cpu")
    cold.load_state_dict(weights)
    assert [cold.step(b) for b in batches[3:]] != want[3:]                  # fresh moments: a different trajectory
    with pytest.raises(SerializationError):
        resumed.load_optimizer_state(opt_tensors, dict(opt_meta, world=2))
    with pytest.raises(SerializationError):
        resumed.load_optimizer_state({"adam.m": opt_tensors["adam.m"]}, opt_meta)
