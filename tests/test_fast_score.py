"""Score-only driver: packing policies, budgets, coverage, end-to-end run on a synthetic cache."""
import json

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from chaoscontrol_b200 import fast_score as FS
from chaoscontrol_b200.eval_stream.io import CachedDoc, load_val_cache, write_synthetic_val_cache
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.runner_exp21 import save_output_ckpt


def _docs(lens):
    out, pos = [], 0
    for i, n in enumerate(lens):
        out.append(CachedDoc(i, pos, n, 3 * n))
        pos += n
    return out


def test_packing_policies_and_rank_split():
    docs = _docs([100, 700, 256, 257, 30, 512])
    assert FS.chunk_count_for_doc(docs[3], chunk_size=256) == 2 and FS.padded_token_work(docs[3], chunk_size=256) == 512
    assert FS.chunk_count_for_doc(docs[0], chunk_size=-1) == 1 and FS.padded_token_work(docs[0], chunk_size=-1) == 100
    assert FS.resolve_doc_packing(doc_packing=None, sort_docs_by_length=None) == "chunk_count_tail"
    assert FS.resolve_doc_packing(doc_packing=None, sort_docs_by_length=False) == "source_order"
    assert FS.resolve_doc_packing(doc_packing="token_len_desc", sort_docs_by_length=False) == "token_len_desc"
    order = lambda p: [w.doc.doc_id for w in FS.prepare_doc_work(docs, doc_packing=p, chunk_size=256)]
    assert order("source_order") == [0, 1, 2, 3, 4, 5]
    assert order("token_len_desc") == [1, 5, 3, 2, 0, 4]
    assert order("chunk_count_desc") == [1, 5, 3, 2, 0, 4]
    assert order("chunk_count_tail")[0] == 1 and set(order("chunk_count_tail")) == set(range(6))
    with pytest.raises(ValueError):
        FS.prepare_doc_work(docs, doc_packing="zigzag", chunk_size=256)
    assert FS.doc_range_for_rank(num_docs=10, rank=1, world_size=3) == (3, 6)
    with pytest.raises(ValueError):
        FS.doc_range_for_rank(num_docs=10, rank=3, world_size=3)
    for packing in ("source_order", "chunk_count_tail"):
        shares = [FS.prepare_rank_doc_work(docs, rank=r, world_size=2, doc_packing=packing, chunk_size=256,
                                           doc_batch_size=1) for r in range(2)]
        ids = sorted(w.doc.doc_id for s in shares for w in s)
        assert ids == list(range(6))
    loads = [sum(FS.padded_token_work(w.doc, chunk_size=256) for w in s) for s in shares]
    assert abs(loads[0] - loads[1]) <= 512


def test_budgets_and_coverage():
    assert FS.resolve_doc_batch_size(requested_doc_batch_size=64, chunk_size=256, max_forward_tokens=4096) == 16
    assert FS.resolve_doc_batch_size(requested_doc_batch_size=64, chunk_size=-1, max_forward_tokens=4096) == 64
    cpu = torch.device("cpu")
    assert FS.resolve_max_forward_tokens(max_forward_tokens=5000, requested_doc_batch_size=4, chunk_size=256, device=cpu) == 5000
    assert FS.resolve_max_forward_tokens(max_forward_tokens="auto", requested_doc_batch_size=4, chunk_size=256, device=cpu) == 1024
    assert FS.resolve_max_forward_tokens(max_forward_tokens="auto", requested_doc_batch_size=4, chunk_size=-1, device=cpu) == 0
    with pytest.raises(ValueError):
        FS.resolve_max_forward_tokens(max_forward_tokens=0, requested_doc_batch_size=4, chunk_size=256, device=cpu)
    assert FS.expected_scored_tokens(token_len=600, chunk_size=256, score_boundary_targets=True) == 599
    assert FS.expected_scored_tokens(token_len=600, chunk_size=256, score_boundary_targets=False) == 597
    assert FS.expected_scored_tokens(token_len=513, chunk_size=256, score_boundary_targets=False) == 510
    assert FS.expected_scored_tokens(token_len=1, chunk_size=256, score_boundary_targets=True) == 0
    d = CachedDoc(7, 0, 600, 1800)
    FS.validate_doc_score_coverage(doc=d, tokens_scored=599, chunk_size=256, score_boundary_targets=True)
    with pytest.raises(RuntimeError, match="coverage mismatch"):
        FS.validate_doc_score_coverage(doc=d, tokens_scored=598, chunk_size=256, score_boundary_targets=True)
    assert FS.record_order_safe_reason(persistence_mode="reset", score_only_mode=True, doc_packing="token_len_desc") \
        == "reset_score_only_commutative_ce_reduction"
    assert FS.record_order_safe_reason(persistence_mode="carry_state", score_only_mode=True,
                                       doc_packing="token_len_desc").startswith("not_order_safe")
    m = CareStudentLM(vocab_size=32, dim=16, num_layers=1)
    assert FS.estimate_max_forward_tokens(m, device=cpu) == FS.DEFAULT_MAX_FORWARD_TOKENS


def test_run_end_to_end_matches_full_sequence_scoring(tmp_path):
    torch.manual_seed(0)
    cache_dir = tmp_path / "val"
    write_synthetic_val_cache(cache_dir, n_docs=12, vocab=48, median_len=40.0, sigma=0.6, min_len=8, max_len=120, seed=3)
    model = CareStudentLM(vocab_size=48, dim=16, num_layers=2)
    cfg = dict(vocab_size=48, model_dim=16, num_layers=2)
    save_output_ckpt(str(tmp_path / "m.pt"), model, cfg)
    out = tmp_path / "o" / "score.json"
    s = FS.run(cache_dir=str(cache_dir), checkpoint_path=str(tmp_path / "m.pt"), output_path=str(out), chunk_size=16,
               doc_batch_size=4, device=torch.device("cpu"))
    cache = load_val_cache(cache_dir)
    ce = 0.0
    for d in cache.iter_docs():
        t = torch.as_tensor(np.asarray(cache.tokens_for(d)).astype(np.int64)).view(1, -1) if hasattr(cache, "tokens_for") \
            else torch.as_tensor(np.asarray(cache.tokens[d.token_start:d.token_start + d.token_len]).astype(np.int64)).view(1, -1)
        with torch.no_grad():
            lg = model(t[:, :-1])["logits"]
        ce += float(F.cross_entropy(lg.reshape(-1, 48), t[:, 1:].reshape(-1), reduction="sum"))
    assert s["docs_scored"] == 12 and s["tokens_scored"] == cache.total_tokens - 12
    assert s["total_ce_nats"] == pytest.approx(ce, rel=1e-4)
    assert s["bpb"] == pytest.approx(ce / np.log(2) / cache.total_raw_bytes, rel=1e-4)
    saved = json.loads(out.read_text())
    assert saved["provenance"]["checkpoint_sha256"] and saved["doc_packing"] == "chunk_count_tail"
    assert FS.main(["--cache-dir", str(cache_dir), "--checkpoint-path", str(tmp_path / "m.pt"), "--chunk-size", "16",
                    "--max-docs", "5", "--max-forward-tokens", "64"]) == 0


@pytest.mark.gpu
def test_graph_chunk_scorer_matches_eager():
    from chaoscontrol_b200.ops import _lib
    from chaoscontrol_b200.scoring import _chunk_loss_rows
    torch.manual_seed(1)
    model = CareStudentLM(vocab_size=512, dim=256, num_layers=2).cuda().to(torch.bfloat16).eval()
    g = FS.GraphChunkScorer(model, batch_size=8, chunk_size=64, device=torch.device("cuda"))
    blk1 = torch.randint(0, 512, (8, 65), device="cuda")
    blk2 = torch.randint(0, 512, (8, 65), device="cuda")
    with torch.no_grad():
        r1, f1 = _chunk_loss_rows(model, blk1[:, :-1].contiguous(), blk1[:, 1:].contiguous(), None)
        r2, f2 = _chunk_loss_rows(model, blk2[:, :-1].contiguous(), blk2[:, 1:].contiguous(), [f.float() for f in f1])
    gr1, gf1 = g.replay(blk1)
    gr1, gf1 = gr1.clone(), [f.clone().float() for f in gf1]
    gr2, gf2 = g.replay(blk2, gf1)
    torch.cuda.synchronize()
    _lib.assert_ok()
    assert torch.equal(gr1, r1) and torch.equal(gr2, r2)
    assert all(torch.equal(a.float(), b.float()) for a, b in zip(gf2, f2))


@pytest.mark.gpu
def test_graph_ttt_matches_the_eager_ttt_driver():
    """Same documents, same SGD rule: the graph-replayed chunk step gives the eager driver's CE."""
    import numpy as np
    from chaoscontrol_b200.eval_stream.types import DocRecord
    from chaoscontrol_b200.models.model import CareStudentLM
    from chaoscontrol_b200.scoring import run_ttt_eval, run_ttt_eval_graph
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    model = CareStudentLM(vocab_size=1024, dim=256, num_layers=2).to(dev).to(torch.bfloat16)
    rng = np.random.default_rng(0)
    docs = [DocRecord(doc_id=i, tokens=rng.integers(0, 1024, n).tolist(), raw_bytes=4 * n)
            for i, n in enumerate([300, 513, 40, 1025, 257])]
    before = [p.detach().clone() for p in model.parameters()]
    kw = dict(adapt_set="log_a+delta_proj", chunk_size=256, eval_lr=0.01)
    fast = run_ttt_eval_graph(model, docs, **kw)
    for p, b in zip(model.parameters(), before):
        assert torch.equal(p, b) and p.requires_grad            # weights restored, flags restored
    slow = run_ttt_eval(model, docs, persistence_mode="reset", steps_per_chunk=1, optimizer="sgd", **kw)
    assert fast["docs_scored"] == 5 and fast["chunks_scored"] == slow["chunks_scored"] == 2 + 2 + 1 + 4 + 1
    assert fast["graph_replays"] == 10 and fast["padded_chunks"] == 2          # tails of 300 and 40 tokens
    assert abs(fast["mean_ce"] - slow["mean_ce"]) < 2e-2 * slow["mean_ce"]
    # adaptation is really happening: a score-only pass gives a different CE on the multi-chunk documents
    none = run_ttt_eval_graph(model, docs, adapt_set="none", chunk_size=256, eval_lr=0.01)
    assert none["adapt_steps"] == 0 and abs(none["per_doc_ce"][3] - fast["per_doc_ce"][3]) > 1e-3
    assert abs(none["per_doc_ce"][2] - fast["per_doc_ce"][2]) < 1e-3 * abs(none["per_doc_ce"][2])
