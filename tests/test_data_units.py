"""Data pipeline, tokenizer, symbol table and metrics logger: one test per component
(the unit tests of crates/data, crates/symbolic and crates/metrics)."""
import io
import struct

import numpy as np
import pytest

from rustral_b200.data import (BOS, EOS, PAD, UNK, DataLoader, DataLoaderConfig, InMemoryDataset, MmapDataset, StreamingDataset,
                               WordLevelConfig, WordLevelTokenizer, shuffled_loader, simple_loader)
from rustral_b200.metrics import ConsoleLogger, MetricsBackend, MetricsLogger, ProgressBar
from rustral_b200.symbolic import Vocabulary


# ---- tokenizer ------------------------------------------------------------------------------------------------------
def test_vocabulary_order_is_frequency_then_alphabet_after_the_specials():
    tok = WordLevelTokenizer.fit_from_iter(["b a a c", "c b a", "d"])
    assert tok.vocab.tokens == [PAD, UNK, BOS, EOS, "a", "b", "c", "d"]         # a:3, b:2, c:2 (tie: alphabet), d:1
    assert (tok.vocab.pad_id, tok.vocab.unk_id, tok.vocab.bos_id, tok.vocab.eos_id) == (0, 1, 2, 3)


def test_min_freq_and_max_vocab_limit_the_vocabulary():
    texts = ["a a a b b c"]
    assert WordLevelTokenizer.fit_from_iter(texts, WordLevelConfig(min_freq=2)).vocab.tokens[4:] == ["a", "b"]
    assert WordLevelTokenizer.fit_from_iter(texts, WordLevelConfig(max_vocab=5)).vocab.tokens[4:] == ["a"]   # specials count


def test_encode_decode_unknowns_case_and_specials():
    tok = WordLevelTokenizer.fit_from_iter(["Hello world"])
    assert tok.encode("hello WORLD again") == [4, 5, 1]
    assert tok.encode_with_specials("world") == [2, 5, 3]
    assert tok.decode([2, 4, 5, 0, 3]) == "hello world" and tok.decode([4, 99]) == f"hello {UNK}"
    cased = WordLevelTokenizer.fit_from_iter(["Hello hello"], WordLevelConfig(lowercase=False))
    assert len(cased.vocab) == 6 and cased.encode("Hello") != cased.encode("hello")


def test_vocab_file_round_trip_and_validation(tmp_path):
    tok = WordLevelTokenizer.fit_from_iter(["x y y"])
    path = tmp_path / "vocab.txt"
    tok.save_vocab(str(path))
    again = WordLevelTokenizer.from_vocab_file(str(path))
    assert again.vocab.tokens == tok.vocab.tokens and again.encode("y x z") == tok.encode("y x z")
    bad = tmp_path / "bad.txt"
    bad.write_text("a\nb\n")
    with pytest.raises(ValueError):
        WordLevelTokenizer.from_vocab_file(str(bad))


# ---- datasets and loaders -------------------------------------------------------------------------------------------
def test_simple_loader_batches_in_order_with_a_short_last_batch():
    loader = simple_loader(list(range(10)), batch_size=4)
    assert loader.num_batches() == 3
    assert [loader.next_batch() for _ in range(3)] == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9]] and loader.next_batch() is None
    loader.reset()
    assert list(loader) == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9]]


def test_shuffled_loader_is_a_seeded_permutation_that_changes_per_epoch():
    a, b, c = (shuffled_loader(list(range(20)), 5, seed=s) for s in (1, 1, 2))
    ea, eb, ec = list(a), list(b), list(c)
    assert ea == eb and ea != ec
    assert sorted(x for batch in ea for x in batch) == list(range(20))
    a.reset()
    assert list(a) != ea                                                         # a new epoch reshuffles
    full = DataLoader(InMemoryDataset(list(range(10))), DataLoaderConfig(4, drop_last=True))
    assert full.num_batches() == 2 and [len(x) for x in full] == [4, 4]


def test_streaming_dataset_reads_lines_lazily(tmp_path):
    p = tmp_path / "lines.txt"
    p.write_text("3\n1\n4\n1\n5\n")
    ds = StreamingDataset(str(p), parse=int)
    assert len(ds) == 5 and ds.get(2) == 4 and ds.get(4) == 5 and ds.get_batch([0, 3]) == [3, 1]
    with pytest.raises(IndexError):
        ds.get(5)


def test_mmap_dataset_serves_fixed_size_records(tmp_path):
    p = tmp_path / "recs.bin"
    vals = np.arange(12, dtype=np.float32)
    p.write_bytes(vals.tobytes())
    ds = MmapDataset(str(p), element_size=12)                                    # three floats per record
    assert len(ds) == 4 and struct.unpack("3f", ds.get(1)) == (3.0, 4.0, 5.0)
    assert ds.get_f32_slice(3).tolist() == [9.0, 10.0, 11.0]
    ds.close()


# ---- symbol table ---------------------------------------------------------------------------------------------------
def test_symbol_table_ids_are_insert_ordered_and_frozen_tables_map_to_unk():
    v = Vocabulary.with_specials("<unk>", ["pos", "neg"])
    assert v.tokens() == ["<unk>", "pos", "neg"] and v.insert("pos") == 1 and v.insert("neutral") == 3
    assert v.id("neg") == 2 and v.id("nope") is None and v.id_or_unk("nope") == 0 and v.token(3) == "neutral" and v.token(9) is None
    v.freeze()
    assert v.is_frozen() and v.insert("late") == 0 and len(v) == 4 and "late" not in v and "pos" in v


# ---- metrics --------------------------------------------------------------------------------------------------------
class _Capture(MetricsBackend):
    def __init__(self):
        self.scalars, self.hists, self.flushes = [], [], 0

    def log_scalar(self, m):
        self.scalars.append((m.name, m.value, m.step))

    def log_histogram(self, m):
        self.hists.append(m)

    def flush(self):
        self.flushes += 1


def test_metrics_logger_fans_out_with_the_current_step():
    a, b = _Capture(), _Capture()
    log = MetricsLogger([a])
    log.add_backend(b)
    log.log_scalar("loss", 2.0)
    log.step(); log.step()
    log.log_scalar("loss", 1.5)
    log.log_scalar_with_step("acc", 0.25, 40)
    log.set_step(7)
    log.log_scalar("lr", 0.1)
    want = [("loss", 2.0, 0), ("loss", 1.5, 2), ("acc", 0.25, 40), ("lr", 0.1, 7)]
    assert a.scalars == want and b.scalars == want
    log.log_training_summary(3, 0.9, accuracy=0.5, lr=0.01)
    assert a.scalars[-3:] == [("train/loss", 0.9, 3), ("train/accuracy", 0.5, 3), ("train/lr", 0.01, 3)] and a.flushes == 1


def test_histograms_bin_the_values():
    cap = _Capture()
    log = MetricsLogger([cap])
    log.log_histogram("w", [0.0, 0.1, 0.2, 0.9, 1.0], bins=2)
    h = cap.hists[0]
    assert h.name == "w" and h.counts == [3, 2] and h.edges == pytest.approx([0.0, 0.5, 1.0])


def test_console_logger_and_progress_bar_write_text():
    out = io.StringIO()
    log = MetricsLogger([ConsoleLogger(flush_every=1, file=out)])
    log.log_scalar("loss", 0.125)
    log.flush()
    assert "loss" in out.getvalue() and "0.125" in out.getvalue()
    bar_out = io.StringIO()
    bar = ProgressBar(4, width=8, file=bar_out)
    bar.update(2, "half")
    bar.update(2)
    text = bar_out.getvalue()
    assert "[####....] 2/4" in text and "[########] 4/4" in text and "half" in text


def test_pinned_batch_prefetcher_serves_batches_in_order_and_blocks_when_full():
    import time

    import torch
    from rustral_b200.data.datasets import PinnedBatchPrefetcher
    made = []

    def make(step):
        made.append(step)
        return torch.full((4,), float(step))
    pf = PinnedBatchPrefetcher(make, depth=2)
    try:
        time.sleep(0.35)                      # the producer fills the queue (2), holds one more batch and waits on the full queue
        assert len(made) == 3
        assert [float(pf.next()[0]) for _ in range(5)] == [0.0, 1.0, 2.0, 3.0, 4.0]
    finally:
        pf.close()
