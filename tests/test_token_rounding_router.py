"""Token-rounding router (host logic, CPU): every expert's load becomes a multiple of the row tile, by trimming its
lowest-scored top-K picks ("down") or by adding the best-scored tokens that did not pick it ("up"); scores are the
renormalised top-K probabilities for picks and the plain softmax probability for additions
(reference: benchmarks/moe-token-rounding.py:139-181)."""
import pytest
import torch

from sonicmoe.routing import token_rounding_routing


@pytest.mark.parametrize("routing", ["down", "up", "nr"])
@pytest.mark.parametrize("T,E,K,tile", [(1024, 16, 4, 128), (512, 8, 8, 128), (2048, 32, 2, 64)])
def test_token_rounding_invariants(routing, T, E, K, tile):
    g = torch.Generator().manual_seed(T + E)
    logits = torch.randn(T, E, generator=g)
    s, tok, exp = token_rounding_routing(logits, K, tile, routing)
    assert tok.dtype == torch.int32 and exp.dtype == torch.int32 and s.dtype == torch.float32
    assert bool((tok[1:] >= tok[:-1]).all()), "pairs are sorted by token"
    pairs = set(zip(tok.tolist(), exp.tolist()))
    assert len(pairs) == tok.numel(), "no duplicate pair"
    counts = torch.bincount(exp.long(), minlength=E)
    assert bool((counts % tile == 0).all())
    probs = torch.softmax(logits, -1)
    tv, ti = probs.topk(K, dim=-1)
    tv = tv / tv.sum(-1, keepdim=True)
    tc = {(t, int(e)): float(v) for t in range(T) for e, v in zip(ti[t].tolist(), tv[t].tolist())}
    tc_counts = torch.bincount(ti.flatten(), minlength=E)
    for e in range(E):
        mine = {t for t, ee in pairs if ee == e}
        picked = {t for (t, ee) in tc if ee == e}
        want = int(tc_counts[e])
        if routing == "down":
            assert counts[e] == want // tile * tile and mine <= picked
        elif routing == "up":
            assert counts[e] == min(-(-want // tile) * tile, T) and (picked <= mine or counts[e] == T)
        if mine and picked - mine:      # trimmed: everything kept scores at least as high as anything dropped
            assert min(tc[(t, e)] for t in mine & picked) >= max(tc[(t, e)] for t in picked - mine) - 1e-7
        if mine - picked:               # added: by plain softmax probability, best first
            added = [float(probs[t, e]) for t in mine - picked]
            rest = [float(probs[t, e]) for t in set(range(T)) - mine - picked]
            assert not rest or min(added) >= max(rest) - 1e-7
    for (t, e), v in zip(zip(tok.tolist(), exp.tolist()), s.tolist()):
        ref = tc[(t, e)] if (t, e) in tc else float(probs[t, e])
        assert abs(v - ref) < 1e-6
