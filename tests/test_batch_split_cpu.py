"""Batch-split schedule: every layer runs the batch as micro-batches; the numbers must not change."""
import pytest
import torch

from helpers import batch_of, tiny_config


def _step(model, extra):
  from maxtext_b200.train.engine import TrainEngine
  cfg = tiny_config(model, ["per_device_batch_size=4", "max_target_length=32", "learning_rate=1e-3"] + extra)
  eng = TrainEngine(cfg, None, torch.device("cpu"))
  b = batch_of(cfg)
  out = [eng.train_step(dict(b)) for _ in range(2)]
  return [float(m["learning/loss"]) for m in out], float(out[0]["learning/raw_grad_norm"]), eng


@pytest.mark.parametrize("model,extra", [("llama2-7b", []), ("deepseek2-16b", ["load_balance_loss_weight=0.0"]),
                                         ("llama2-7b", ["remat_policy=minimal_with_context"]), ("gemma2-2b", [])])
def test_split_layers_reproduce_the_unsplit_step(model, extra):
  base, gn0, _ = _step(model, extra)
  split, gn1, eng = _step(model, extra + ["use_batch_split_schedule=true"])
  assert eng.config.use_batch_split_schedule
  assert abs(base[0] - split[0]) < 1e-5 * max(1.0, abs(base[0])), (base, split)
  assert abs(gn0 - gn1) < 1e-4 * max(1.0, gn0), (gn0, gn1)
  assert abs(base[1] - split[1]) < 1e-4 * max(1.0, abs(base[1])), (base, split)


def test_auxiliary_losses_are_averaged_over_micro_batches():
  base, _, _ = _step("deepseek2-16b", ["load_balance_loss_weight=0.01"])
  split, _, _ = _step("deepseek2-16b", ["load_balance_loss_weight=0.01", "use_batch_split_schedule=true", "batch_split_factor=4"])
  # the balance loss is not linear in the batch, so the two differ a little, but stay on the same scale
  assert abs(base[0] - split[0]) < 5e-2 * abs(base[0]), (base, split)


def test_micro_context_slices_rows_and_keeps_its_own_store():
  from maxtext_b200.layers.context import LayerCtx
  pos = torch.arange(8)[None].expand(4, 8)
  seg = torch.arange(4)[:, None].expand(4, 8) + 1
  ctx = LayerCtx(None, pos, seg, tokens=torch.arange(32).view(4, 8), saved={}, save_names=("context",))
  a, b = ctx.micro(0, 2), ctx.micro(1, 2)
  assert a.positions.shape == (2, 8) and b.segment_ids[0, 0] == 3 and b.tokens[0, 0] == 16 and b.micro_slot == 1 and b.batch_split == 1
  a.keep("context", torch.ones(1))
  b.keep("context", torch.zeros(1))
  assert set(ctx.saved) == {"mb0", "mb1"} and float(ctx.saved["mb0"]["context"]) == 1.0 and float(ctx.saved["mb1"]["context"]) == 0.0
  a.aux_losses.append(("x", torch.ones(())))
  assert ctx.aux_losses == [] and b.aux_losses == []
