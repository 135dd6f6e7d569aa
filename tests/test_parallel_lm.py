"""The parallel decoder LM (dense and mixture-of-experts) on one device: training reduces the loss on CPU, and the GPU
kernels give the same loss and gradients as the CPU reference path."""
import pytest
import torch

from rustral_b200.models.parallel_lm import MixedPrecisionAdamW, ParallelDecoderLM, ParallelLMConfig


def _cfg(moe: bool):
    return ParallelLMConfig(vocab_size=256, d_model=64, n_layer=2, n_head=2, n_kv_head=1, ffn_hidden=128, seq_len=32,
                            num_experts=4 if moe else 0, top_k=2)


@pytest.mark.parametrize("moe", [False, True])
def test_parallel_lm_trains_on_cpu(moe):
    cfg = _cfg(moe)
    model = ParallelDecoderLM(cfg, "cpu", seed=1)
    opt = MixedPrecisionAdamW(model, lr=3e-3, weight_decay=0.0)
    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len + 1), generator=g)
    losses = []
    for _ in range(8):
        loss = model.forward_loss(tokens)
        loss.backward()
        opt.accumulate()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0] - 0.2, losses
    assert cfg.num_params() > 0 and cfg.flops_per_token() > 0


@pytest.mark.gpu
@pytest.mark.parametrize("moe", [False, True])
def test_parallel_lm_gpu_matches_cpu(moe):
    cfg = ParallelLMConfig(vocab_size=512, d_model=128, n_layer=2, n_head=2, n_kv_head=1, ffn_hidden=256, seq_len=128,
                           num_experts=4 if moe else 0, top_k=2)
    cpu = ParallelDecoderLM(cfg, "cpu", seed=3)
    gpu = ParallelDecoderLM(cfg, "cuda", seed=3)
    for n, p in cpu.params.items():            # same weights on both devices
        gpu.params[n].data.copy_(p.data)
    tokens = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len + 1), generator=torch.Generator().manual_seed(5))
    lc = cpu.forward_loss(tokens)
    lc.backward()
    lg = gpu.forward_loss(tokens.cuda())
    lg.backward()
    assert abs(float(lc.detach()) - float(lg.detach())) < 3e-2, (float(lc.detach()), float(lg.detach()))
    for n in ("l0.wqkv", "l1.wo", "wte", "head"):
        a, b = gpu.params[n].grad.float().cpu(), cpu.params[n].grad.float()
        assert (a - b).norm() / (b.norm() + 1e-9) < 8e-2, n


def test_parallel_lm_loads_hugging_face_llama_and_shards_it_for_tensor_parallelism():
    """A Llama built by `transformers` -> utils.hf -> ParallelDecoderLM: the training loss equals Hugging Face's (bf16
    parameters, so to about 1e-2); the tensor-parallel shards of a two-rank layout tile the full tensors exactly; a
    state_dict round trip is lossless."""
    transformers = pytest.importorskip("transformers")
    from rustral_b200.parallel.process_group import ProcessGroup
    from rustral_b200.utils.hf import convert_hf_llama
    torch.manual_seed(0)
    lc = transformers.LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32, rope_theta=10000.0,
                                  rms_norm_eps=1e-5, tie_word_embeddings=False, attention_dropout=0.0)
    hf = transformers.LlamaForCausalLM(lc).eval()
    state = convert_hf_llama(hf.state_dict())
    cfg = ParallelLMConfig(vocab_size=256, d_model=64, n_layer=2, n_head=4, n_kv_head=2, ffn_hidden=128, seq_len=32,
                           rope_theta=10000.0, eps=1e-5)
    model = ParallelDecoderLM(cfg, "cpu", seed=9)
    model.load_state_dict(state)
    tokens = torch.randint(0, 256, (3, 33), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(tokens[:, :-1], labels=None).logits.float()
        ref_loss = torch.nn.functional.cross_entropy(ref.reshape(-1, 256), tokens[:, 1:].reshape(-1))
        loss = model.forward_loss(tokens)
    assert abs(float(loss) - float(ref_loss)) < 2e-2, (float(loss), float(ref_loss))
    from rustral_b200.utils.hf import export_hf_llama
    exported = export_hf_llama(state)                       # and back into transformers: names and values round-trip
    ref_sd = {k: v for k, v in hf.state_dict().items() if "rotary_emb" not in k}
    assert set(exported) == set(ref_sd) and all(torch.equal(exported[k], ref_sd[k].float()) for k in ref_sd)
    hf.load_state_dict(exported, strict=False)
    back = model.state_dict()
    assert set(back) == set(state)
    for k in state:
        assert torch.equal(back[k], state[k].bfloat16().float()), k
    with pytest.raises(KeyError):
        model.load_state_dict({k: v for k, v in state.items() if k != "layers.1.ffn.down.weight"})
    with pytest.raises(ValueError):
        model.load_state_dict(dict(state, **{"final_norm.weight": torch.ones(3)}))
    # two tensor-parallel ranks: the shards tile the full tensors
    groups = ProcessGroup.new_threaded(2)
    shards = []
    for pg in groups:
        m = ParallelDecoderLM(cfg, "cpu", tp_pg=pg, seed=9)
        m.load_state_dict(state)
        shards.append(m.params)
    hd, full = 16, model.params
    q0, q1 = shards[0]["l0.wqkv"], shards[1]["l0.wqkv"]
    assert torch.equal(torch.cat([q0[:2 * hd], q1[:2 * hd]]), full["l0.wqkv"][:4 * hd])                 # query heads
    assert torch.equal(torch.cat([q0[2 * hd:3 * hd], q1[2 * hd:3 * hd]]), full["l0.wqkv"][4 * hd:6 * hd])  # key heads
    assert torch.equal(torch.cat([shards[0]["l1.wo"], shards[1]["l1.wo"]], 1), full["l1.wo"])
    assert torch.equal(torch.cat([shards[0]["l1.wdown"], shards[1]["l1.wdown"]], 1), full["l1.wdown"])
    assert torch.equal(torch.cat([shards[0]["l0.wgu"][:64], shards[1]["l0.wgu"][:64]]), full["l0.wgu"][:128])
    assert torch.equal(torch.cat([shards[0]["head"], shards[1]["head"]]), full["head"])
    assert torch.equal(shards[1]["wte"], full["wte"])


def test_tensor_parallel_shards_gather_back_into_the_full_checkpoint():
    """load_state_dict (shard) and gather_state_dict (collective reassembly) are inverses on two tensor-parallel ranks,
    and a tensor-parallel forward of the loaded model gives the single-rank loss."""
    import threading
    from rustral_b200.parallel.process_group import ProcessGroup
    cfg = ParallelLMConfig(vocab_size=256, d_model=64, n_layer=2, n_head=4, n_kv_head=2, ffn_hidden=128, seq_len=32)
    full = ParallelDecoderLM(cfg, "cpu", seed=4)
    state = full.state_dict()
    tokens = torch.randint(0, 256, (2, 33), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want = float(full.forward_loss(tokens))
    groups = ProcessGroup.new_threaded(2)
    results, errors = [None, None], []

    def worker(i):
        try:
            m = ParallelDecoderLM(cfg, "cpu", tp_pg=groups[i], seed=77)
            m.load_state_dict(state)
            with torch.no_grad():
                loss = float(m.forward_loss(tokens))
            results[i] = (m.gather_state_dict(), loss)
        except Exception as e:      # noqa: BLE001
            errors.append(e)
    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not errors, errors
    for gathered, loss in results:
        assert set(gathered) == set(state) and abs(loss - want) < 2e-2
        for k in state:
            assert torch.equal(gathered[k], state[k]), k
