"""Property tests (hypothesis): invariants that must hold for any input, not just the hand-picked ones."""
import torch
from hypothesis import given, settings, strategies as st

from rustral_b200.io import safetensors_io as sio
from rustral_b200.nn import PagedCache
from rustral_b200.parallel.checkpoint import reshard_flat
from rustral_b200.parallel.compression import CompressionType, ErrorFeedbackCompression

_DT = [torch.float32, torch.bfloat16, torch.float16, torch.int64, torch.int32, torch.uint8, torch.bool]


@settings(max_examples=40, deadline=None)
@given(st.lists(st.tuples(st.text("abcxyz._0", min_size=1, max_size=8), st.sampled_from(range(len(_DT))),
                          st.lists(st.integers(0, 5), min_size=0, max_size=3), st.integers(0, 1000)), min_size=0, max_size=6))
def test_safetensors_round_trip_of_arbitrary_state(entries):
    state = {}
    for name, di, shape, seed in entries:
        dt = _DT[di]
        g = torch.Generator().manual_seed(seed)
        t = torch.randint(0, 2, shape, generator=g).to(dt) if not dt.is_floating_point else (torch.randn(shape, generator=g) * 10).to(dt)
        state[name] = t
    back, meta = sio.deserialize(sio.serialize(state, {"n": len(state)}))
    assert set(back) == set(state) and meta == {"n": str(len(state))}
    for k, t in state.items():
        assert back[k].dtype == t.dtype and back[k].shape == t.shape and torch.equal(back[k], t)


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 200), st.integers(1, 8), st.integers(1, 8))
def test_resharding_a_flat_buffer_keeps_every_element_in_order(n, old_world, new_world):
    full = torch.arange(float(n))
    per = (n + old_world - 1) // old_world
    padded = torch.cat([full, torch.zeros(per * old_world - n)])
    old = [padded[r * per:(r + 1) * per] for r in range(old_world)]
    new = [reshard_flat(old, new_world, r) for r in range(new_world)]
    assert len({s.numel() for s in new}) == 1                      # equal shards
    joined = torch.cat(new)
    assert torch.equal(joined[:n], full) and float(joined[n:].abs().sum()) == 0.0


@settings(max_examples=40, deadline=None)
@given(st.lists(st.tuples(st.integers(0, 5), st.integers(1, 40), st.booleans()), min_size=1, max_size=40))
def test_paged_cache_never_loses_or_shares_a_block(ops):
    blocks, bs = 12, 4
    c = PagedCache(blocks, bs, allocate_storage=False)
    want = {}                                                       # sequence -> tokens it may hold
    for seq, tokens, free in ops:
        if free:
            c.free(seq)
            want.pop(seq, None)
        else:
            before = c.free_blocks
            ok = c.allocate(seq, tokens)
            if ok:
                want[seq] = max(want.get(seq, 0), tokens)
            else:
                assert c.free_blocks == before                     # a refused request changes nothing
        tables = {s: c.block_table(s) for s in want}
        used = [b for t in tables.values() for b in t]
        assert len(used) == len(set(used)) and all(0 <= b < blocks for b in used)            # no block is shared
        assert c.free_blocks + len(used) == blocks                                            # none is lost
        assert all(len(tables[s]) == (want[s] + bs - 1) // bs for s in want) and c.num_sequences() == len(want)
    for s in list(want):
        c.free(s)
    assert c.free_blocks == blocks


@settings(max_examples=25, deadline=None)
@given(st.sampled_from([CompressionType.ONE_BIT, CompressionType.FOUR_BIT, CompressionType.FP8, CompressionType.BF16]),
       st.integers(1, 12), st.integers(0, 10_000))
def test_error_feedback_conserves_the_sum_of_what_was_sent(kind, steps, seed):
    g = torch.Generator().manual_seed(seed)
    ef = ErrorFeedbackCompression(kind)
    true = torch.zeros(64, dtype=torch.float64)
    sent = torch.zeros(64, dtype=torch.float64)
    for _ in range(steps):
        x = torch.randn(64, generator=g)
        true += x.double()
        sent += ef.compress(x).double()
    assert torch.allclose(true, sent + ef.residual.double(), atol=1e-4)      # nothing is dropped: it is sent or still owed


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 60), st.integers(1, 9), st.booleans(), st.booleans(), st.integers(0, 5))
def test_a_loader_epoch_visits_every_item_once(n, batch, shuffle, drop_last, seed):
    from rustral_b200.data.datasets import DataLoader, DataLoaderConfig, InMemoryDataset
    items = list(range(n))
    mk = lambda: DataLoader(InMemoryDataset(items), DataLoaderConfig(batch, shuffle, seed, 0, drop_last))
    loader = mk()
    epochs = [[b for b in loader] for _ in range(3)]
    for batches in epochs:
        flat = [x for b in batches for x in b]
        kept = n - n % batch if drop_last else n
        assert len(flat) == kept and len(set(flat)) == kept and set(flat) <= set(items)
        assert all(len(b) == batch for b in batches[:-1]) and (not batches or 0 < len(batches[-1]) <= batch)
        assert len(batches) == loader.num_batches()
        if not shuffle:
            assert flat == items[:kept]
    assert [[b for b in mk()] for _ in range(1)][0] == epochs[0]                  # same seed, same first epoch
    if shuffle and n >= 8 and not drop_last:
        orders = [[x for b in e for x in b] for e in epochs]
        assert orders[0] != orders[1] or orders[1] != orders[2]                  # reshuffled between epochs


@settings(max_examples=50, deadline=None)
@given(st.lists(st.lists(st.sampled_from(["alpha", "Beta", "gamma", "delta", "x", "y1", "Zed"]), min_size=0, max_size=8), min_size=1, max_size=8),
       st.integers(0, 9))
def test_word_tokenizer_round_trips_known_words_and_honours_the_vocabulary_cap(docs, cap):
    import os
    import tempfile
    from rustral_b200.data.tokenizer import WordLevelConfig, WordLevelTokenizer
    texts = [" ".join(d) for d in docs]
    tok = WordLevelTokenizer.fit_from_iter(texts, WordLevelConfig(lowercase=True, max_vocab=cap))
    v = tok.vocab
    assert len(v.tokens) >= 4 and len(set(v.tokens[:4])) == 4 and [v.pad_id, v.unk_id, v.bos_id, v.eos_id] == [0, 1, 2, 3]
    if cap:
        assert len(v) <= max(cap, 4)
    words = sorted({w.lower() for d in docs for w in d})
    if cap == 0:
        assert set(v.tokens[4:]) == set(words)
        for t in texts:
            assert tok.decode(tok.encode(t)) == " ".join(t.lower().split())
    for t in texts:
        ids = tok.encode_with_specials(t)
        assert ids[0] == v.bos_id and ids[-1] == v.eos_id and all(0 <= i < len(v) for i in ids)
        assert tok.decode(ids) == tok.decode(tok.encode(t))                        # specials are dropped by decode
    assert tok.encode("neverseenword") == [v.unk_id]
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "vocab.txt")
        tok.save_vocab(path)
        again = WordLevelTokenizer.from_vocab_file(path)
        assert again.vocab.tokens == v.tokens and all(again.encode(t) == tok.encode(t) for t in texts)


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 12), st.integers(2, 8), st.integers(0, 1000), st.booleans())
def test_top_k_routing_invariants(tokens, experts, seed, renorm):
    from rustral_b200.ops import moe
    k = min(2, experts)
    logits = torch.randn(tokens, experts, generator=torch.Generator().manual_seed(seed))
    idx, w, probs = moe.route(logits, k, renorm)
    assert idx.shape == (tokens, k) and torch.allclose(probs.sum(-1), torch.ones(tokens), atol=1e-6)
    assert all(len(set(row)) == k for row in idx.tolist())                         # distinct experts per token
    top = probs.topk(k, -1).values
    picked = probs.gather(1, idx.long())
    assert torch.allclose(picked, top, atol=1e-7)                                   # the k most probable ones, in order
    if renorm:
        assert torch.allclose(w.sum(-1), torch.ones(tokens), atol=1e-6)
    else:
        assert torch.allclose(w, picked, atol=1e-7)


@settings(max_examples=80, deadline=None)
@given(st.integers(0, 40), st.integers(1, 9))
def test_stage_splitting_covers_every_layer_once_and_leaves_no_stage_idle_when_it_need_not(layers, stages):
    from rustral_b200.parallel.pipeline_parallel import StageSplitter
    parts = StageSplitter.split_by_count(layers, stages)
    assert len(parts) == stages and [i for p in parts for i in p] == list(range(layers))         # contiguous cover
    sizes = [len(p) for p in parts]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    if layers >= stages:
        assert min(sizes) >= 1


@settings(max_examples=60, deadline=None)
@given(st.lists(st.integers(1, 1000), min_size=1, max_size=24), st.integers(1, 6))
def test_parameter_balanced_splitting_is_a_contiguous_cover(counts, stages):
    from rustral_b200.parallel.pipeline_parallel import StageSplitter
    parts = StageSplitter.balance_by_params(counts, stages)
    assert len(parts) == stages and [i for p in parts for i in p] == list(range(len(counts)))
    if len(counts) >= stages:
        assert all(parts[s] for s in range(stages))          # no empty stage when there are enough layers
