"""Command line for the SGNS embedding pipeline:

``python -m chaoscontrol_b200.sgns.cli train``          skip-gram negative-sampling training on the train shards
                                                     (scripts/train_sgns.py:26-109)
``python -m chaoscontrol_b200.sgns.cli prepare-inits``  the family of ``embed.weight`` initialisers derived from one
                                                     trained table (scripts/prepare_sgns_inits.py:70-257)
``python -m chaoscontrol_b200.sgns.cli report``         intrinsic quality numbers of a table
                                                     (scripts/sgns_intrinsic_report.py:35-110)
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import Optional, Sequence

import torch

from .intrinsic import kmeans_clusters, nearest_neighbors
from .model import SGNSModel
from .moment_match import (frequency_bucket_ids, match_full_covariance, match_row_norm_moments,
                           sample_full_covariance, sample_with_row_norms, shuffle_rows,
                           shuffle_rows_within_buckets, token_class_bucket_ids)
from .sampler import NegativeSampler, unigram_probs_from_counts
from .train import train_one_epoch

__all__ = ["main", "subsample_frequent", "derive_inits"]


def subsample_frequent(stream: torch.Tensor, counts: torch.Tensor, threshold: float, *,
                       generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Word2vec subsampling: token ``w`` survives with probability
    ``min(1, sqrt(t / f(w)) + t / f(w))`` where ``f`` is its relative frequency."""
    if threshold <= 0:
        return stream
    f = counts.double() / counts.sum().clamp_min(1)
    keep = (torch.sqrt(threshold / f.clamp_min(1e-30)) + threshold / f.clamp_min(1e-30)).clamp(max=1.0).float()
    u = torch.rand(stream.shape, generator=generator)
    return stream[u < keep[stream.long()]]


def _train(a: argparse.Namespace) -> int:
    from ..data import load_fineweb_tokens
    torch.manual_seed(a.seed)
    train, _ = load_fineweb_tokens(a.data_dir)
    stream = train[: a.max_tokens].to(torch.int64).clamp_(0, a.vocab_size - 1)
    counts = torch.bincount(stream, minlength=a.vocab_size)
    g = torch.Generator().manual_seed(a.seed)
    stream = subsample_frequent(stream, counts, a.subsample_threshold, generator=g)
    dev = torch.device(a.device)
    model = SGNSModel(vocab_size=a.vocab_size, dim=a.dim).to(dev)
    sampler = NegativeSampler(unigram_probs_from_counts(counts.float()))
    opt = torch.optim.SGD(model.parameters(), lr=a.lr)
    stream = stream.to(dev)
    history = []
    for epoch in range(a.epochs):
        loss = train_one_epoch(model, stream, sampler, a.window, a.k, a.batch_size, opt, max_batches=a.max_batches)
        history.append(loss)
        print(f"[sgns] epoch {epoch + 1}/{a.epochs} loss {loss:.4f} tokens {stream.numel():,}", flush=True)
    a.out.parent.mkdir(parents=True, exist_ok=True)
    torch.save(model.input_embed.weight.detach().float().cpu(), a.out)
    a.out.with_suffix(".json").write_text(json.dumps({
        "vocab_size": a.vocab_size, "dim": a.dim, "window": a.window, "k": a.k, "epochs": a.epochs,
        "batch_size": a.batch_size, "lr": a.lr, "subsample_threshold": a.subsample_threshold,
        "tokens_after_subsampling": int(stream.numel()), "loss_history": history, "seed": a.seed}, indent=2))
    return 0


def derive_inits(sgns: torch.Tensor, *, reference_seed: int = 0, shuffled_seed: int = 42, norm_seed: int = 101,
                 norm_shuffled_seed: int = 102, fullcov_shuffled_seed: int = 103, random_fullcov_seed: int = 104,
                 token_counts: Optional[torch.Tensor] = None, freq_buckets: int = 8, freq_shuffled_seed: int = 105,
                 pieces: Optional[Sequence[str]] = None, class_shuffled_seed: int = 106) -> dict[str, torch.Tensor]:
    """Every initialiser of the embedding-init study from one trained table.  The
    reference cloud is the model's default embedding init (unit Gaussian)."""
    V, D = sgns.shape
    ref = torch.randn(V, D, generator=torch.Generator().manual_seed(reference_seed))
    meanstd = match_row_norm_moments(sgns.float(), ref)
    fullcov = match_full_covariance(sgns.float(), ref)
    out = {"meanstd": meanstd, "fullcov": fullcov, "shuffled": shuffle_rows(meanstd, shuffled_seed),
           "zero": torch.zeros(V, D), "norm_only": sample_with_row_norms(meanstd, seed=norm_seed),
           "norm_only_shuffled": sample_with_row_norms(meanstd, seed=norm_seed,
                                                       shuffle_norms_seed=norm_shuffled_seed),
           "fullcov_shuffled": shuffle_rows(fullcov, fullcov_shuffled_seed),
           "random_fullcov": sample_full_covariance(fullcov, seed=random_fullcov_seed)}
    if token_counts is not None:
        ids = frequency_bucket_ids(token_counts, num_buckets=freq_buckets)
        out["freq_bucket_shuffle"] = shuffle_rows_within_buckets(meanstd, ids, seed=freq_shuffled_seed)
    if pieces is not None:
        out["class_bucket_shuffle"] = shuffle_rows_within_buckets(meanstd, token_class_bucket_ids(pieces),
                                                                 seed=class_shuffled_seed)
    return out


def _prepare(a: argparse.Namespace) -> int:
    sgns = torch.load(a.sgns, map_location="cpu", weights_only=True)
    if sgns.dim() != 2:
        raise SystemExit(f"--sgns must hold a (vocab, dim) tensor, got shape {tuple(sgns.shape)}")
    V = sgns.shape[0]
    counts = None
    if a.token_counts is not None:
        counts = torch.load(a.token_counts, map_location="cpu", weights_only=True).reshape(-1)
        if counts.numel() != V:
            raise SystemExit(f"--token-counts has {counts.numel()} entries for a vocabulary of {V}")
    elif a.data_dir_for_counts is not None:
        from ..data import load_fineweb_tokens
        train, _ = load_fineweb_tokens(str(a.data_dir_for_counts))
        counts = torch.bincount(train[: a.counts_max_tokens].to(torch.int64).clamp_(0, V - 1), minlength=V)
    pieces = None
    if a.sp_model is not None:
        import sentencepiece as spm
        sp = spm.SentencePieceProcessor()
        sp.Load(str(a.sp_model))
        pieces = [sp.id_to_piece(i) if i < sp.vocab_size() else "" for i in range(V)]
    inits = derive_inits(sgns, reference_seed=a.reference_seed, shuffled_seed=a.shuffled_seed,
                         norm_seed=a.norm_seed, norm_shuffled_seed=a.norm_shuffled_seed,
                         fullcov_shuffled_seed=a.fullcov_shuffled_seed, random_fullcov_seed=a.random_fullcov_seed,
                         token_counts=counts, freq_buckets=a.freq_buckets, freq_shuffled_seed=a.freq_shuffled_seed,
                         pieces=pieces, class_shuffled_seed=a.class_shuffled_seed)
    out_dir = Path(a.out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    for name, t in inits.items():
        path = out_dir / f"sgns_init_{name}.pt"
        torch.save(t.contiguous(), path)
        print(f"[sgns] {path} shape {tuple(t.shape)} row-norm mean {float(t.norm(dim=-1).mean()):.4f}", flush=True)
    return 0


def _random_pair_mean_cos(embed: torch.Tensor, n_pairs: int, seed: int) -> float:
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(0, embed.shape[0], (n_pairs,), generator=g)
    b = torch.randint(0, embed.shape[0], (n_pairs,), generator=g)
    e = torch.nn.functional.normalize(embed.float(), dim=-1)
    return float((e[a] * e[b]).sum(-1).mean())


def _report(a: argparse.Namespace) -> int:
    embed = torch.load(a.embed, map_location="cpu", weights_only=True).float()
    decode = str
    if a.sp_model is not None:
        import sentencepiece as spm
        sp = spm.SentencePieceProcessor()
        sp.Load(str(a.sp_model))
        decode = lambda i: sp.id_to_piece(int(i)) if int(i) < sp.vocab_size() else f"<{int(i)}>"   # noqa: E731
    queries = list(range(min(a.n_common, embed.shape[0])))
    nn_ids = nearest_neighbors(embed, queries, k=a.k_nn)
    e = torch.nn.functional.normalize(embed, dim=-1)
    nn_cos = float(torch.stack([(e[q] @ e[torch.tensor(v)].T).mean() for q, v in nn_ids.items()]).mean())
    clusters = kmeans_clusters(embed, a.k_clusters)
    sizes = torch.bincount(clusters, minlength=a.k_clusters).tolist()
    report = {"vocab_size": int(embed.shape[0]), "dim": int(embed.shape[1]),
              "row_norm_mean": float(embed.norm(dim=-1).mean()), "row_norm_std": float(embed.norm(dim=-1).std()),
              "random_pair_mean_cos": _random_pair_mean_cos(embed, a.n_random_pairs, a.seed),
              "nearest_neighbor_mean_cos": nn_cos, "cluster_sizes": sizes,
              "neighbors": {decode(q): [decode(v) for v in vs] for q, vs in list(nn_ids.items())[:10]}}
    text = json.dumps(report, indent=2, ensure_ascii=False)
    if a.out is not None:
        a.out.write_text(text)
    print(text)
    return 0


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="chaoscontrol_b200.sgns.cli", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    t = sub.add_parser("train", help="train an SGNS table on the training shards")
    t.add_argument("--data-dir", required=True)
    t.add_argument("--vocab-size", type=int, required=True)
    t.add_argument("--dim", type=int, default=256)
    t.add_argument("--window", type=int, default=5)
    t.add_argument("--k", type=int, default=10)
    t.add_argument("--epochs", type=int, default=3)
    t.add_argument("--batch-size", type=int, default=4096)
    t.add_argument("--lr", type=float, default=0.025)
    t.add_argument("--subsample-threshold", type=float, default=1e-5)
    t.add_argument("--max-tokens", type=int, default=50_000_000)
    t.add_argument("--max-batches", type=int, default=None)
    t.add_argument("--out", type=Path, required=True)
    t.add_argument("--seed", type=int, default=0)
    t.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    t.set_defaults(fn=_train)
    p = sub.add_parser("prepare-inits", help="derive the embedding initialisers from a trained table")
    p.add_argument("--sgns", required=True)
    p.add_argument("--out-dir", required=True)
    p.add_argument("--reference-seed", type=int, default=0)
    p.add_argument("--shuffled-seed", type=int, default=42)
    p.add_argument("--norm-seed", type=int, default=101)
    p.add_argument("--norm-shuffled-seed", type=int, default=102)
    p.add_argument("--fullcov-shuffled-seed", type=int, default=103)
    p.add_argument("--random-fullcov-seed", type=int, default=104)
    p.add_argument("--token-counts", type=Path, default=None)
    p.add_argument("--data-dir-for-counts", type=Path, default=None)
    p.add_argument("--counts-max-tokens", type=int, default=50_000_000)
    p.add_argument("--freq-buckets", type=int, default=8)
    p.add_argument("--freq-shuffled-seed", type=int, default=105)
    p.add_argument("--sp-model", type=Path, default=None)
    p.add_argument("--class-shuffled-seed", type=int, default=106)
    p.set_defaults(fn=_prepare)
    r = sub.add_parser("report", help="intrinsic quality report of a table")
    r.add_argument("--embed", type=Path, required=True)
    r.add_argument("--sp-model", type=Path, default=None)
    r.add_argument("--n-common", type=int, default=50)
    r.add_argument("--k-clusters", type=int, default=20)
    r.add_argument("--k-nn", type=int, default=5)
    r.add_argument("--n-random-pairs", type=int, default=20000)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", type=Path, default=None)
    r.set_defaults(fn=_report)
    a = ap.parse_args(argv)
    return int(a.fn(a))


if __name__ == "__main__":
    raise SystemExit(main())
