"""Generation: cached decode equals cache-free decode token for token; filters behave."""

import pytest
import torch

from kohakuwullm_b200.generation.engine import (LocalGenerator, advance, filter_min_p, filter_top_k, filter_top_p,
                                                sample)
from kohakuwullm_b200.models import LMBackbone, get_preset


@pytest.fixture()
def wide_model():
    # a wide init makes greedy decoding non-degenerate, so the comparison below can actually fail
    torch.manual_seed(0)
    cfg = get_preset("B200-smoke", vocab_size=97, dim=64, depth=2, heads=2, kv_heads=1, head_dim=32, mlp_hidden=128,
                     init_std=0.3, sliding_window=4, global_layer_every=2, attn_sink=True, attn_num_sinks=2)
    return LMBackbone(cfg)


def test_cached_decode_matches_cache_free(wide_model):
    prompt = torch.randint(0, 97, (3, 5))
    a = LocalGenerator(wide_model, eos_id=96, use_cache=True).generate(prompt, 12, temperature=0.0)
    b = LocalGenerator(wide_model, eos_id=96, use_cache=False).generate(prompt, 12, temperature=0.0)
    assert torch.equal(a, b)
    assert len(set(a[0, 5:].tolist())) > 1, "degenerate decode: the comparison proves nothing"


def test_filters():
    logits = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    assert torch.isinf(filter_top_k(logits, 2)[0, :2]).all() and torch.isfinite(filter_top_k(logits, 2)[0, 2:]).all()
    kept = torch.isfinite(filter_top_p(logits, 0.6))[0]
    assert kept.tolist() == [False, False, False, True] or kept.tolist() == [False, False, True, True]
    assert torch.isfinite(filter_min_p(logits, 0.5))[0].tolist() == [False, False, False, True]
    assert sample(logits, temperature=0.0).item() == 3
    with pytest.raises(FloatingPointError):
        sample(torch.full((1, 4), float("nan")))


def test_finished_rows_hold_eos():
    tokens = torch.zeros(2, 1, dtype=torch.long)
    finished = torch.tensor([True, False])
    tokens, finished = advance(tokens, torch.tensor([5, 7]), finished, (7,), eos=9)
    assert tokens[:, -1].tolist() == [9, 7] and finished.tolist() == [True, True]
