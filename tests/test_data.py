"""Indexed token files, GPT samples and the per-rank batch iterator (CPU)."""
import json
import struct

import numpy as np
import pytest
import torch

from kareus_b200.data import (GPTDataset, GPTDatasetConfig, IndexedDataset, IndexedDatasetWriter, PretrainingBatches,
                              build_sample_index, split_documents)
from kareus_b200.data import preprocess


def _corpus(tmp_path, n_docs=120, vocab=500, seed=0, dtype=np.uint16, empty_every=0):
    rng = np.random.RandomState(seed)
    docs = [rng.randint(0, vocab, size=rng.randint(1, 60)) for _ in range(n_docs)]
    if empty_every:
        for i in range(0, n_docs, empty_every):
            docs[i] = np.zeros(0, dtype=np.int64)
    prefix = str(tmp_path / "corpus_text_document")
    with IndexedDatasetWriter(prefix, dtype=dtype) as w:
        w.add_documents(docs)
    return prefix, docs


def test_index_file_layout_and_round_trip(tmp_path):
    prefix, docs = _corpus(tmp_path)
    raw = open(prefix + ".idx", "rb").read()
    assert raw[:9] == b"MMIDIDX\x00\x00"
    version, = struct.unpack("<Q", raw[9:17])
    code, = struct.unpack("<B", raw[17:18])
    n_seq, n_doc = struct.unpack("<QQ", raw[18:34])
    assert (version, code, n_seq, n_doc) == (1, 8, len(docs), len(docs) + 1)      # code 8: uint16
    assert len(raw) == 34 + 4 * n_seq + 8 * n_seq + 8 * n_doc
    ds = IndexedDataset(prefix)
    assert len(ds) == len(docs) and ds.num_documents == len(docs)
    assert ds.num_tokens == sum(len(d) for d in docs)
    for i in (0, 7, len(docs) - 1):
        np.testing.assert_array_equal(ds[i], docs[i])
    np.testing.assert_array_equal(ds.get(7, 1, 2), docs[7][1:3]) if len(docs[7]) >= 3 else None
    with pytest.raises(IndexError):
        ds.get(0, 0, len(docs[0]) + 1)
    np.testing.assert_array_equal(ds.document_lengths(), [len(d) for d in docs])


def test_documents_of_several_sequences(tmp_path):
    prefix = str(tmp_path / "s")
    with IndexedDatasetWriter(prefix, dtype=np.int32) as w:
        w.add_sequence([1, 2, 3]); w.add_sequence([4, 5]); w.end_document()
        w.add_document([6, 7, 8, 9])
    ds = IndexedDataset(prefix)
    assert len(ds) == 3 and ds.num_documents == 2
    np.testing.assert_array_equal(ds.document_lengths(), [5, 4])
    g = GPTDataset(ds, GPTDatasetConfig(seq_len=4, num_samples=2, seed=0, shuffle_samples=False))
    stream = np.concatenate([[1, 2, 3, 4, 5] if d == 0 else [6, 7, 8, 9] for d in g.doc_order])
    np.testing.assert_array_equal(g.sample_tokens(0), stream[0:5])
    np.testing.assert_array_equal(g.sample_tokens(1), stream[4:9])


@pytest.mark.parametrize("empty_every", [0, 5])
def test_samples_cut_the_shuffled_stream(tmp_path, empty_every):
    prefix, docs = _corpus(tmp_path, empty_every=empty_every)
    ds = IndexedDataset(prefix)
    seq, n = 32, 400                      # more than one epoch of this corpus
    g = GPTDataset(ds, GPTDatasetConfig(seq_len=seq, num_samples=n, seed=11, shuffle_samples=False))
    assert g.num_epochs >= 2
    # every epoch is a permutation of all documents
    per_epoch = g.doc_order.reshape(g.num_epochs, -1)
    for row in per_epoch:
        assert sorted(row.tolist()) == list(range(len(docs)))
    stream = np.concatenate([docs[d] for d in g.doc_order])
    for i in (0, 1, 57, n - 1):
        np.testing.assert_array_equal(g.sample_tokens(i), stream[i * seq:(i + 1) * seq + 1])
    item = g[3]
    assert item["tokens"].shape == (seq,) and item["labels"].shape == (seq,) and item["tokens"].dtype == torch.int64
    torch.testing.assert_close(item["tokens"][1:], item["labels"][:-1])       # labels are the inputs shifted by one
    # native walker and the numpy statement agree, also with empty documents in the stream
    a = build_sample_index(ds.document_lengths(), g.doc_order, seq, n, native=False)
    np.testing.assert_array_equal(a, g.sample_index)
    with pytest.raises(ValueError):
        build_sample_index(ds.document_lengths(), g.doc_order[:3], seq, n)


def test_sample_order_is_a_seeded_permutation_and_masks_eod(tmp_path):
    prefix, _ = _corpus(tmp_path)
    ds = IndexedDataset(prefix)
    cfg = GPTDatasetConfig(seq_len=16, num_samples=100, seed=5, eod_token=7)
    g1, g2 = GPTDataset(ds, cfg), GPTDataset(ds, cfg)
    assert sorted(g1.shuffle.tolist()) == list(range(100)) and g1.shuffle.tolist() != list(range(100))
    for i in (0, 50, 99):
        torch.testing.assert_close(g1[i]["tokens"], g2[i]["tokens"])
    g3 = GPTDataset(ds, GPTDatasetConfig(seq_len=16, num_samples=100, seed=6))
    assert any(not torch.equal(g1[i]["tokens"], g3[i]["tokens"]) for i in range(10))
    it = g1[0]
    assert torch.equal(it["loss_mask"] == 0, it["tokens"] == 7)
    with pytest.raises(ValueError):
        GPTDataset(ds, GPTDatasetConfig(seq_len=16, num_samples=4, vocab_size=10))[0]


def test_split_documents():
    assert split_documents(1000, (949, 50, 1)) == ((0, 949), (949, 999), (999, 1000))
    assert split_documents(10, (1, 0, 0)) == ((0, 10), (10, 10), (10, 10))
    with pytest.raises(ValueError):
        split_documents(10, (0, 0))


def test_ranks_share_the_global_batch_and_resume(tmp_path):
    prefix, _ = _corpus(tmp_path)
    ds = IndexedDataset(prefix)
    g = GPTDataset(ds, GPTDatasetConfig(seq_len=16, num_samples=96, seed=2))
    mbs, num_mb = 2, 3
    # one rank alone sees the whole global batch of 12 in order
    with PretrainingBatches(g, mbs, num_mb * 2, pin=False) as one:
        whole = [next(one)["tokens"] for _ in range(3)]
        assert one.consumed_samples == 36
    with PretrainingBatches(g, mbs, num_mb, dp_rank=0, dp_size=2, pin=False) as r0, \
            PretrainingBatches(g, mbs, num_mb, dp_rank=1, dp_size=2, pin=False) as r1:
        for step in range(3):
            a, b = next(r0)["tokens"], next(r1)["tokens"]
            assert a.shape == (mbs * num_mb, 16)
            # blocks of micro_batch x dp: rank r holds rows [r*mbs, (r+1)*mbs) of every block
            blocks = whole[step].reshape(num_mb, 2, mbs, 16)
            torch.testing.assert_close(a, blocks[:, 0].reshape(-1, 16))
            torch.testing.assert_close(b, blocks[:, 1].reshape(-1, 16))
    # a run that stopped after two steps continues with the third batch
    with PretrainingBatches(g, mbs, num_mb * 2, consumed_samples=24, pin=False) as again:
        torch.testing.assert_close(next(again)["tokens"], whole[2])
        assert again.steps_left() == (96 - 36) // 12
    # the iterator ends with the data
    with PretrainingBatches(g, mbs, num_mb * 2, consumed_samples=84, pin=False) as last:
        next(last)
        with pytest.raises(StopIteration):
            next(last)
    with pytest.raises(ValueError):
        PretrainingBatches(g, mbs, num_mb, consumed_samples=5, pin=False)


def test_reader_errors_reach_the_training_loop(tmp_path):
    class Broken(torch.utils.data.Dataset):
        def __len__(self):
            return 100

        def __getitem__(self, i):
            raise RuntimeError("disk gone")

    with PretrainingBatches(Broken(), 2, 2, pin=False) as it:
        with pytest.raises(RuntimeError, match="disk gone"):
            next(it)


def test_context_parallel_ranks_get_their_two_chunks(tmp_path):
    from kareus_b200.parallel.collectives import dual_chunk_ids
    prefix, _ = _corpus(tmp_path)
    g = GPTDataset(IndexedDataset(prefix), GPTDatasetConfig(seq_len=32, num_samples=8, seed=2))
    with PretrainingBatches(g, 2, 2, pin=False) as full, PretrainingBatches(g, 2, 2, cp=2, cp_rank=1, pin=False) as part:
        f, p = next(full), next(part)
    a, b = dual_chunk_ids(2, 1)
    c = 32 // 4
    want = torch.cat([f["tokens"][:, a * c:(a + 1) * c], f["tokens"][:, b * c:(b + 1) * c]], dim=1)
    torch.testing.assert_close(p["tokens"], want)
    assert p["loss_mask"].shape == (4, 16)


def test_preprocess_cli(tmp_path):
    src = tmp_path / "c.jsonl"
    texts = ["hello world", "", "energy-aware training", "ü"]
    src.write_text("\n".join(json.dumps({"text": t, "other": "x"}) for t in texts))
    out = str(tmp_path / "wiki")
    assert preprocess.main(["--input", str(src), "--json-keys", "text", "--output-prefix", out, "--append-eod"]) == 0
    ds = IndexedDataset(out + "_text_document")
    assert ds.num_documents == 3                                   # the empty document is dropped
    assert bytes(ds[0][:-1].astype(np.uint8)).decode() == "hello world" and int(ds[0][-1]) == 256
    assert bytes(ds[2][:-1].astype(np.uint8)).decode() == "ü"
    ids = tmp_path / "ids.txt"
    ids.write_text("1 2 3\n4 5\n")
    assert preprocess.main(["--input", str(ids), "--token-ids", "--output-prefix", str(tmp_path / "t"),
                            "--vocab-size", "100000"]) == 0
    t = IndexedDataset(str(tmp_path / "t_text_document"))
    assert t.dtype == np.int32 and t.num_tokens == 5


def test_training_on_a_token_file(tmp_path):
    """run_train reads its batches from an indexed file and a resumed run continues with the next batch."""
    from kareus_b200.cli import run_train
    prefix, _ = _corpus(tmp_path, n_docs=300, vocab=120)
    common = ["--model", "tiny", "--mbs", "2", "--gbs", "4", "--seq", "32", "--method", "nanobatch", "--data-path",
              prefix, "--data-split", "1,0,0", "--out", str(tmp_path / "runs"), "--keep-process-group"]
    assert run_train.main(common + ["--steps", "3", "--save", str(tmp_path / "ck")]) == 0
    assert run_train.main(common + ["--steps", "4", "--load", str(tmp_path / "ck")]) == 0


def test_pretrain_yaml_names_the_token_file(tmp_path, capsys):
    """`model.data.data_prefix` of the reference's YAML layout (a [weight, prefix] blend) selects the token file;
    a prefix that does not exist falls back to synthetic tokens with a note."""
    from kareus_b200.cli import pretrain
    prefix, _ = _corpus(tmp_path, n_docs=300, vocab=200)
    yaml_text = """
name: tiny_data
trainer: {{devices: 1, num_nodes: 1, precision: 32, max_steps: 2}}
model:
  micro_batch_size: 2
  global_batch_size: 4
  encoder_seq_length: 32
  num_layers: 2
  hidden_size: 64
  ffn_hidden_size: 128
  num_attention_heads: 4
  num_query_groups: 2
  vocab_size: 256
  activations_checkpoint_granularity: full
  data:
    data_prefix: [1.0, {prefix}]
    splits_string: 900,50,50
"""
    (tmp_path / "c.yaml").write_text(yaml_text.format(prefix=prefix))
    assert pretrain.main(["--config", str(tmp_path / "c.yaml"), "--out", str(tmp_path / "exp")]) == 0
    out = capsys.readouterr().out
    assert "data: " + prefix in out and "step 1 loss" in out
    (tmp_path / "d.yaml").write_text(yaml_text.format(prefix=str(tmp_path / "missing")))
    assert pretrain.main(["--config", str(tmp_path / "d.yaml"), "--out", str(tmp_path / "exp2")]) == 0
    assert "training on synthetic tokens" in capsys.readouterr().out


def test_validation_loss_on_held_out_documents(tmp_path, capsys):
    from kareus_b200.cli import run_train
    prefix, _ = _corpus(tmp_path, n_docs=400, vocab=120)
    rc = run_train.main(["--model", "tiny", "--mbs", "2", "--gbs", "4", "--seq", "32", "--method", "nanobatch",
                         "--data-path", prefix, "--data-split", "8,2,0", "--steps", "4", "--eval-interval", "2",
                         "--eval-iters", "2", "--out", str(tmp_path / "runs"), "--keep-process-group"])
    assert rc == 0
    out = capsys.readouterr().out
    assert out.count("validation loss") == 2 and "(2 batches)" in out
    # without a token file the held-out batches are synthetic
    rc = run_train.main(["--model", "tiny", "--mbs", "2", "--gbs", "4", "--seq", "32", "--method", "megatron",
                         "--steps", "2", "--eval-interval", "1", "--out", str(tmp_path / "runs2"),
                         "--keep-process-group"])
    assert rc == 0 and capsys.readouterr().out.count("validation loss") == 2


def test_metrics_log(tmp_path):
    from kareus_b200.cli import run_train
    rc = run_train.main(["--model", "tiny", "--mbs", "2", "--gbs", "4", "--seq", "32", "--method", "nanobatch",
                         "--steps", "3", "--eval-interval", "3", "--out", str(tmp_path / "runs"),
                         "--keep-process-group"])
    assert rc == 0
    f = tmp_path / "runs" / "tiny" / "cp1_tp1_mbs2_seq32" / "nanobatch" / "metrics_global_rank-0.jsonl"
    rows = [json.loads(l) for l in f.read_text().splitlines()]
    steps = [r for r in rows if "loss" in r]
    assert [r["step"] for r in steps] == [0, 1, 2] and steps[-1]["consumed_samples"] == 12
    assert all(r["grad_norm"] > 0 and r["lr"] > 0 and r["tokens_per_s"] > 0 for r in steps)
    assert [r for r in rows if "validation_loss" in r][0]["step"] == 2


def test_weighted_blend_of_two_files(tmp_path, capsys):
    from kareus_b200.data import BlendedDataset, build_blend_index
    ds, pos = build_blend_index([1.0, 3.0], 400)
    counts = np.bincount(ds)
    assert counts.tolist() == [100, 300]
    # every prefix of the blend keeps each dataset within one sample of its share
    run = np.cumsum(ds == 0)
    assert np.all(np.abs(run - 0.25 * np.arange(1, 401)) <= 1.0)
    assert pos[ds == 0].tolist() == list(range(100)) and pos[ds == 1].tolist() == list(range(300))
    a, b = build_blend_index([1.0, 3.0], 400, native=False)
    np.testing.assert_array_equal(a, ds)
    np.testing.assert_array_equal(b, pos)

    class Const(torch.utils.data.Dataset):
        def __init__(self, v, n):
            self.v, self.n = v, n

        def __len__(self):
            return self.n

        def __getitem__(self, i):
            assert 0 <= i < self.n
            return (self.v, i)

    blend = BlendedDataset([1.0, 3.0], lambda d, n: Const(d, n), 40)
    got = [blend[i] for i in range(40)]
    assert sum(1 for v, _ in got if v == 0) == 10 and got[0][1] == 0
    # through the driver: two files, 1:3
    from kareus_b200.cli import run_train
    (tmp_path / "a").mkdir(); (tmp_path / "b").mkdir()
    pa, _ = _corpus(tmp_path / "a", n_docs=200, vocab=100, seed=1)
    pb, _ = _corpus(tmp_path / "b", n_docs=200, vocab=100, seed=2)
    rc = run_train.main(["--model", "tiny", "--mbs", "2", "--gbs", "4", "--seq", "32", "--method", "megatron", "--steps",
                         "2", "--data-path", "1", pa, "3", pb, "--data-split", "9,1,0", "--eval-interval", "2", "--out",
                         str(tmp_path / "runs"), "--keep-process-group"])
    out = capsys.readouterr().out
    assert rc == 0 and out.count("data: ") == 2 and "validation loss" in out
