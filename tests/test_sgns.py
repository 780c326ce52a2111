"""SGNS embeddings and moment matching (cf. tests/unit/test_sgns_*.py of the reference)."""
import pytest
import torch
import torch.nn.functional as F

from chaoscontrol_b200 import sgns


def test_nce_loss_matches_definition_and_trains():
    torch.manual_seed(0)
    m = sgns.SGNSModel(20, 8)
    with torch.no_grad():
        m.output_embed.weight.normal_(0, 0.5)
        m.input_embed.weight.normal_(0, 0.5)
    c, ctx, neg = torch.randint(0, 20, (6,)), torch.randint(0, 20, (6,)), torch.randint(0, 20, (6, 3))
    wi, wp, wn = m.input_embed(c), m.output_embed(ctx), m.output_embed(neg)
    ref = (-F.logsigmoid((wi * wp).sum(-1)) - F.logsigmoid(-torch.einsum("bd,bkd->bk", wi, wn)).sum(-1)).mean()
    assert torch.allclose(sgns.nce_loss(m, c, ctx, neg), ref, atol=1e-6)
    assert torch.allclose(m.score_pairs(c, ctx), (wi * wp).sum(-1))
    # two alternating "topics": co-occurring tokens end up closer than tokens of the other topic
    torch.manual_seed(1)
    a = torch.randint(0, 5, (4000,))
    stream = torch.where((torch.arange(4000) // 50) % 2 == 0, a, a + 5)
    model = sgns.SGNSModel(10, 16)
    probs = sgns.unigram_probs_from_counts(torch.bincount(stream, minlength=10))
    opt = torch.optim.Adam(model.parameters(), lr=0.05)
    l0 = sgns.train_one_epoch(model, stream, sgns.NegativeSampler(probs), window=2, k=4, batch_size=256, opt=opt,
                              max_batches=5)
    for _ in range(2):
        l1 = sgns.train_one_epoch(model, stream, sgns.NegativeSampler(probs), window=2, k=4, batch_size=256, opt=opt)
    assert l1 < l0
    nn_ = sgns.nearest_neighbors(model.input_embed.weight.detach(), [0, 7], k=4)
    assert set(nn_[0]) == {1, 2, 3, 4} and set(nn_[7]) == {5, 6, 8, 9}
    labels = sgns.kmeans_clusters(model.input_embed.weight.detach(), 2)
    assert len(set(labels[:5].tolist())) == 1 and labels[0] != labels[5]


def test_pair_iterator_covers_every_pair_once():
    stream = torch.arange(7)
    pairs = sorted((int(c), int(x)) for cb, xb in sgns.iter_center_context_batches(stream, 2, 3)
                   for c, x in zip(cb, xb))
    want = sorted((i, j) for i in range(7) for j in range(7) if i != j and abs(i - j) <= 2)
    assert pairs == want
    assert list(sgns.iter_center_context_batches(stream, 0, 3)) == []
    assert list(sgns.iter_center_context_batches(torch.arange(1), 2, 3)) == []


def test_sampler():
    p = sgns.unigram_probs_from_counts(torch.tensor([16.0, 1.0, 0.0]))
    assert torch.allclose(p, torch.tensor([8.0, 1.0, 0.0]) / 9.0)
    assert torch.allclose(sgns.unigram_probs_from_counts(torch.tensor([5.0, 1.0]), power=0.0), torch.tensor([0.5, 0.5]))
    s = sgns.NegativeSampler(p).sample(50, 4)
    assert s.shape == (50, 4) and int(s.max()) <= 1
    with pytest.raises(AssertionError):
        sgns.NegativeSampler(torch.tensor([0.5, 0.2]))


def test_moment_matching_and_controls():
    torch.manual_seed(2)
    src, tgt = torch.randn(500, 6) * 3, torch.randn(400, 6) @ torch.randn(6, 6) + 2.0
    out = sgns.match_row_norm_moments(src, tgt)
    assert torch.allclose(F.normalize(out, dim=-1), F.normalize(src, dim=-1), atol=1e-5)
    assert torch.allclose(out.norm(dim=-1).mean(), tgt.norm(dim=-1).mean(), rtol=1e-4)
    assert torch.allclose(out.norm(dim=-1).std(), tgt.norm(dim=-1).std(), rtol=1e-3)
    rec = sgns.match_full_covariance(src, tgt)
    assert torch.allclose(torch.cov(rec.T), torch.cov(tgt.T), atol=2e-2, rtol=2e-2)
    assert torch.allclose(rec.mean(0), tgt.mean(0), atol=1e-4)
    syn = sgns.sample_full_covariance(tgt, seed=0)
    assert syn.shape == tgt.shape and torch.allclose(torch.cov(syn.T), torch.cov(tgt.T), atol=5e-2, rtol=5e-2)
    sh = sgns.shuffle_rows(src, 3)
    assert torch.equal(sh, sgns.shuffle_rows(src, 3)) and not torch.equal(sh, src)
    assert torch.allclose(sh.sum(0), src.sum(0), atol=1e-3)
    sw = sgns.sample_with_row_norms(src, seed=1)
    assert torch.allclose(sw.norm(dim=-1), src.norm(dim=-1), rtol=1e-5)
    sw2 = sgns.sample_with_row_norms(src, seed=1, shuffle_norms_seed=4)
    assert torch.allclose(sw2.norm(dim=-1).sort().values, src.norm(dim=-1).sort().values, rtol=1e-5)
    buckets = torch.arange(500) % 3
    wb = sgns.shuffle_rows_within_buckets(src, buckets, seed=5)
    assert not torch.equal(wb, src)
    for b in range(3):
        assert torch.allclose(wb[buckets == b].sum(0), src[buckets == b].sum(0), atol=1e-3)
        assert torch.equal(wb[buckets == b].norm(dim=-1).sort().values, src[buckets == b].norm(dim=-1).sort().values)
    with pytest.raises(ValueError):
        sgns.shuffle_rows_within_buckets(src, buckets[:10], seed=0)
    fb = sgns.frequency_bucket_ids(torch.tensor([1.0, 9.0, 5.0, 7.0]), num_buckets=2)
    assert fb.tolist() == [1, 0, 1, 0]
    with pytest.raises(ValueError):
        sgns.frequency_bucket_ids(torch.ones(3), num_buckets=0)
    assert sgns.token_class_bucket_ids(["▁the", "!?", "42", "abc", "a1", " "]).tolist() == [0, 1, 2, 3, 4, 0]


def test_cli_train_prepare_report(tmp_path):
    import json

    import numpy as np
    from chaoscontrol_b200.sgns import cli
    rng = np.random.default_rng(0)
    rng.integers(0, 32, 6000, dtype=np.uint16).tofile(tmp_path / "fineweb_train_000.bin")
    rng.integers(0, 32, 600, dtype=np.uint16).tofile(tmp_path / "fineweb_val_000.bin")
    table = tmp_path / "art" / "sgns_v32_d8.pt"
    assert cli.main(["train", "--data-dir", str(tmp_path), "--vocab-size", "32", "--dim", "8", "--epochs", "1",
                     "--batch-size", "256", "--max-batches", "4", "--subsample-threshold", "0.05",
                     "--out", str(table), "--device", "cpu"]) == 0
    w = torch.load(table, weights_only=True)
    assert w.shape == (32, 8) and json.loads(table.with_suffix(".json").read_text())["epochs"] == 1
    assert cli.main(["prepare-inits", "--sgns", str(table), "--out-dir", str(tmp_path / "inits"),
                     "--data-dir-for-counts", str(tmp_path), "--freq-buckets", "4"]) == 0
    names = sorted(p.stem.removeprefix("sgns_init_") for p in (tmp_path / "inits").glob("*.pt"))
    assert names == sorted(["meanstd", "fullcov", "shuffled", "zero", "norm_only", "norm_only_shuffled",
                            "fullcov_shuffled", "random_fullcov", "freq_bucket_shuffle"])
    ms = torch.load(tmp_path / "inits" / "sgns_init_meanstd.pt", weights_only=True)
    sh = torch.load(tmp_path / "inits" / "sgns_init_shuffled.pt", weights_only=True)
    assert torch.allclose(ms.norm(dim=-1).sort().values, sh.norm(dim=-1).sort().values, atol=1e-5)
    assert not torch.equal(ms, sh) and float(torch.load(tmp_path / "inits" / "sgns_init_zero.pt").abs().sum()) == 0
    out = tmp_path / "report.json"
    assert cli.main(["report", "--embed", str(table), "--n-common", "8", "--k-clusters", "3", "--k-nn", "2",
                     "--n-random-pairs", "100", "--out", str(out)]) == 0
    rep = json.loads(out.read_text())
    assert rep["vocab_size"] == 32 and sum(rep["cluster_sizes"]) == 32 and -1 <= rep["random_pair_mean_cos"] <= 1
    # subsampling keeps rare tokens and thins frequent ones
    stream = torch.cat([torch.zeros(9000, dtype=torch.long), torch.arange(1, 11)])
    kept = cli.subsample_frequent(stream, torch.bincount(stream, minlength=11), 1e-3,
                                  generator=torch.Generator().manual_seed(0))
    assert (kept != 0).sum() == 10 and (kept == 0).sum() < 2000
