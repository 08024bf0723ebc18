"""The plain implementation itself: properties that do not need the engine (no GPU)."""
import math

import numpy as np
import torch

from helpers import CONFIGS, random_tokens
from plain import qwen2_plain as P
from plain import sampling_plain as S


def test_rms_norm_and_silu():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = P.rms_norm(x, torch.tensor([1.0, 2.0], dtype=torch.float64), 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[3 / r, 8 / r]], dtype=torch.float64))
    assert abs(float(P.silu(torch.tensor(0.0))) - 0.0) < 1e-12
    assert abs(float(P.silu(torch.tensor(2.0, dtype=torch.float64))) - 2 / (1 + math.exp(-2))) < 1e-12


def test_rope_is_a_rotation_of_split_halves():
    x = torch.randn(5, 3, 8, dtype=torch.float64)
    pos = torch.tensor([0, 1, 2, 50, 51])
    y = P.rope_neox(x, pos, 10000.0)
    assert torch.allclose(y[0], x[0])                                   # position 0: identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    # pair (0, 4) of head 0 at position 1 turns by 1 radian (freq_0 = 1)
    a, b = float(x[1, 0, 0]), float(x[1, 0, 4])
    assert abs(float(y[1, 0, 0]) - (a * math.cos(1) - b * math.sin(1))) < 1e-9
    assert abs(float(y[1, 0, 4]) - (a * math.sin(1) + b * math.cos(1))) < 1e-9
    # scores depend on the distance only
    q = torch.randn(1, 1, 8, dtype=torch.float64).expand(5, 1, 8)
    k = torch.randn(1, 1, 8, dtype=torch.float64).expand(5, 1, 8)
    rq, rk = P.rope_neox(q, pos, 10000.0), P.rope_neox(k, pos, 10000.0)
    assert abs(float((rq[1] * rk[0]).sum() - (rq[4] * rk[3]).sum())) < 1e-6


def test_attention_mask_groups_and_window():
    T, nh, nkv, hd = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n, hd, dtype=torch.float64) for n in (nh, nkv, nkv))
    o = P.causal_attention(q, k, v)
    assert torch.allclose(o[0, 0], v[0, 0]) and torch.allclose(o[0, 3], v[0, 1])    # first row = V[0] of its group
    v2 = v.clone(); v2[5:] += 1.0
    assert torch.allclose(P.causal_attention(q, k, v2)[:5], o[:5])                  # no look-ahead
    w = P.causal_attention(q, k, v, window=3)
    assert torch.allclose(w[:3], o[:3]) and not torch.allclose(w[5], o[5])
    v3 = v.clone(); v3[:4] += 7.0                                                   # keys 0..3 are outside for rows >= 6
    assert torch.allclose(P.causal_attention(q, k, v3, window=3)[6:], w[6:])
    assert not torch.allclose(P.causal_attention(q, k, v3, window=3)[5], w[5])      # row 5 still sees key 3


def test_whole_model_prefix_property_and_tie(folders):
    for name in ("A", "B", "C"):
        m = P.PlainModel(folders(name))
        toks = random_tokens(CONFIGS[name]["vocab_size"], 40, 11)
        full = m.logits(toks)
        assert full.shape == (40, CONFIGS[name]["vocab_size"]) and torch.isfinite(full).all()
        assert torch.allclose(m.logits(toks[:17]), full[:17], atol=1e-10)
        assert ("lm_head.weight" in m.tensors) == (not CONFIGS[name]["tie_word_embeddings"])
    c = P.PlainModel(folders("C"))
    assert [P.layer_window(c.cfg, i) for i in range(4)] == [None, None, 24, 24]


def test_greedy_takes_the_highest_index_of_equal_maxima():
    assert S.greedy(torch.tensor([1.0, 5.0, 5.0, 2.0])) == 2


def test_lcg_and_sampler():
    u = [float(S.lcg_unit(S.draw_seed(S.DEFAULT_SEED, 0, d))) for d in range(200)]
    assert all(0.0 <= x <= 1.0 for x in u) and 0.4 < np.mean(u) < 0.6
    logits = torch.tensor([0.0, 3.0, 1.0, 2.9, -5.0])
    picks = [S.sample(logits, 1.0, 1.0, 0, S.draw_seed(1, 0, d)) for d in range(300)]
    assert set(picks) <= {0, 1, 2, 3, 4} and picks.count(1) > picks.count(2) > 0
    assert {S.sample(logits, 1.0, 1.0, 2, s) for s in range(100)} == {1, 3}          # top-k 2
    assert {S.sample(logits, 1.0, 0.3, 0, s) for s in range(100)} == {1}             # nucleus of one
    assert {S.sample(logits, 1e-9, 1.0, 0, s) for s in range(20)} == {1}             # temperature clamps, no NaN
    assert S.sample(logits, 0.0, 0.5, 3, 1) == 1                                    # 0 = greedy


def test_plain_loop_reasons():
    f = lambda toks: torch.nn.functional.one_hot(torch.tensor((toks[-1] + 1) % 50), 50).float()
    assert S.generate(f, [1], max_tokens=3) == ([2, 3, 4], "max_tokens")
    assert S.generate(f, [1], max_tokens=9, stop_ids=[4]) == ([2, 3], "stop_token")
    assert S.generate(f, [1, 2, 3], max_tokens=9, max_seq=5) == ([4, 5], "context_full")
    assert S.generate(f, [1], max_tokens=0) == ([], "max_tokens")
