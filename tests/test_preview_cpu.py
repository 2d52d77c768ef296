"""Preview prompts cut from the trained batch, the router-bias schedule and the sample preview callback."""

import torch

from kohakuwullm_b200.data.packing import collate_packed
from kohakuwullm_b200.data.preview import batch_documents, prompts_from_batch, trained_spans
from kohakuwullm_b200.models import LMBackbone, get_preset
from kohakuwullm_b200.training.parallel.uwupipe_callbacks import RouterBiasSchedule, SamplePreview


def _chat_doc(n_prompt, n_answer, base):
    ids = torch.arange(base, base + n_prompt + n_answer)
    mask = torch.ones_like(ids, dtype=torch.bool)
    mask[:n_prompt] = False           # the user turn is not trained
    return ids, mask


def test_turn_cut_comes_from_the_loss_mask():
    docs = [_chat_doc(7, 5, 100), _chat_doc(3, 9, 200), torch.arange(300, 340)]
    batch = collate_packed(docs)
    got = batch_documents(batch)
    assert [d[0].numel() for d in got] == [12, 12, 40]
    assert trained_spans(got[0][1]) == [(7, 12)]
    prompts = prompts_from_batch(batch, 5, seed=1)
    assert len(prompts) == 2 and all(name.startswith("batch/turn/") for name, _ in prompts)
    # what the pipeline loaders hand out (a step of several packs) is read the same way as a list of packs
    from kohakuwullm_b200.data.loader.iterative import MicroBatchedStep

    step = MicroBatchedStep([batch, collate_packed([_chat_doc(4, 4, 400)])])
    assert [d[0].numel() for d in batch_documents(step)] == [12, 12, 40, 8]
    assert len(prompts_from_batch(step, 5, seed=1)) == 3
    by_first = {int(p[0]): p for _, p in prompts}
    assert by_first[100].tolist() == list(range(100, 107))
    assert by_first[200].tolist() == list(range(200, 203))
    # plain documents join only when asked for, cut at the fraction; draws are seeded
    more = prompts_from_batch(batch, 5, seed=1, turns_only=False, prefix_frac=0.25)
    plain = [p for n, p in more if n.startswith("batch/prefix/")]
    assert len(plain) == 1 and plain[0].tolist() == list(range(300, 310))
    assert [n for n, _ in prompts_from_batch(batch, 5, seed=1)] == [n for n, _ in prompts]


def _moe_model():
    torch.manual_seed(0)
    cfg = get_preset("B200-smoke", vocab_size=300, dim=64, depth=2, heads=2, kv_heads=1, head_dim=32, mlp_hidden=128,
                     moe_every=1, moe_first_dense=0, moe_num_experts=4, moe_top_k=2, moe_hidden=64)
    return LMBackbone(cfg)


def test_router_bias_schedule_scales_the_built_rate_without_compounding():
    model = _moe_model()
    cb = RouterBiasSchedule(model, lambda step: 0.0 if step < 2 else 0.5)

    class Loop:
        global_step = 0

    cb.on_train_start(Loop())
    routers = [m for m in model.modules() if hasattr(m, "expert_bias")]
    built = cb.base[0]
    assert all(r.bias_update_rate == 0.0 for r in routers)
    for step in (1, 2, 3, 4):
        Loop.global_step = step
        cb.on_train_batch_end(Loop())
    assert all(abs(r.bias_update_rate - 0.5 * built) < 1e-12 for r in routers)
    again = RouterBiasSchedule(model, lambda step: 2.0)
    again.load_state_dict(cb.state_dict())
    again.apply(10)
    assert abs(routers[0].bias_update_rate - 2.0 * built) < 1e-12


def test_sample_preview_reports_rows_on_schedule():
    from kohakuwullm_b200.data import ByteTokenizer

    model = _moe_model()
    seen = []
    cb = SamplePreview(model, ByteTokenizer(), [("greeting", "hi there")], every_n_steps=2, samples=2,
                       max_new_tokens=5, report=lambda step, rows: seen.append((step, rows)))

    class Loop:
        global_step = 0

    cb.on_train_start(Loop())                     # throwaway validation decode: reported nowhere
    assert seen == []
    for step in (1, 2, 3, 4):
        Loop.global_step = step
        cb.on_train_batch_end(Loop())
    assert [s for s, _ in seen] == [2, 4]
    rows = seen[0][1]
    assert len(rows) == 2 and rows[0][0] == "greeting" and rows[0][1] == "hi there" and isinstance(rows[0][3], str)
