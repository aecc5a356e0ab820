"""Post-training: objective weights reproduce autograd gradients; SFT / DPO / GRPO / distillation steps run and move
the quantities they should."""
import torch

from helpers import make_engine, tiny_config
from maxtext_b200.trainers.post_train import objectives as O
from maxtext_b200.trainers.post_train import trainers as T


def test_dpo_weights_equal_autograd_of_the_loss():
  torch.manual_seed(0)
  B, S, beta = 3, 5, 0.3
  lc = torch.randn(B, S, requires_grad=True)       # token losses (-log pi) of chosen / rejected
  lr = torch.randn(B, S, requires_grad=True)
  mc, mr = (torch.rand(B, S) > 0.3).float(), (torch.rand(B, S) > 0.3).float()
  ref_c, ref_r = torch.randn(B), torch.randn(B)
  pi_c, pi_r = O.sequence_logprob(lc, mc), O.sequence_logprob(lr, mr)
  loss, wc, wr, _ = O.dpo_weights(pi_c.detach(), pi_r.detach(), ref_c, ref_r, mc, mr, beta)
  full = -torch.nn.functional.logsigmoid(beta * ((pi_c - pi_r) - (ref_c - ref_r)))
  full.sum().backward()
  assert torch.allclose(lc.grad, wc, atol=1e-6) and torch.allclose(lr.grad, wr, atol=1e-6)
  assert torch.allclose(loss, full.detach(), atol=1e-6)


def test_grpo_weights_equal_autograd_of_the_clipped_surrogate():
  torch.manual_seed(1)
  N, S = 4, 6
  old = torch.randn(N, S)
  new = (old + 0.3 * torch.randn(N, S)).requires_grad_(True)
  adv = O.grpo_advantages(torch.tensor([1.0, 0.0, 3.0, 2.0]), 2)
  mask = torch.ones(N, S)
  ratio = torch.exp(old - new)
  sur = -(torch.minimum(ratio * adv[:, None], ratio.clamp(0.8, 1.2) * adv[:, None]) * mask).sum() / mask.sum()
  sur.backward()
  _, w = O.grpo_weights(new.detach(), old, adv, mask, 0.2)
  assert torch.allclose(new.grad * mask.sum(), w, atol=1e-5)      # engine divides by the normaliser (= mask.sum())
  assert abs(adv.view(2, 2).mean(1)).max() < 1e-6


def test_sft_step_trains_only_on_completions():
  cfg = tiny_config("llama3-8b", ["sft_train_on_completion_only=true", "learning_rate=5e-3"])
  eng = make_engine(cfg)
  prompts = [[5, 6, 7, 8], [9, 10, 11]]
  comps = [[20, 21, 22], [30, 31, 32, 33]]
  losses = [float(T.sft_step(eng, prompts, comps)["learning/loss"]) for _ in range(6)]
  assert losses[-1] < losses[0]
  m = T.sft_step(eng, prompts, comps)
  assert int(m["learning/total_weights"]) == 7             # 3 + 4 completion tokens


def test_dpo_trainer_raises_the_margin():
  cfg = tiny_config("llama3-8b", ["learning_rate=2e-3"])
  eng = make_engine(cfg)
  tr = T.DPOTrainer(eng, beta=0.5)
  prompts, chosen, rejected = [[3, 4, 5]] * 2, [[10, 11, 12]] * 2, [[20, 21, 22]] * 2
  first = tr.step(prompts, chosen, rejected)
  for _ in range(5):
    last = tr.step(prompts, chosen, rejected)
  assert float(last["dpo/loss"]) < float(first["dpo/loss"]) and float(last["dpo/reward_accuracy"]) == 1.0


def test_grpo_trainer_increases_reward_of_a_toy_task():
  torch.manual_seed(0)
  cfg = tiny_config("llama3-8b", ["learning_rate=5e-3", "vocab_size=32", "max_prefill_predict_length=8", "gradient_clipping_threshold=1.0"])
  eng = make_engine(cfg)
  reward = lambda p, c: sum(1.0 for t in c if t % 2 == 0) / len(c)      # likes even tokens
  tr = T.GRPOTrainer(eng, reward, group_size=4, max_new_tokens=6)
  r = [float(tr.step([[1, 2, 3], [4, 5]])["rl/mean_reward"]) for _ in range(12)]
  assert sum(r[-4:]) / 4 > sum(r[:4]) / 4


def test_distillation_step_pulls_student_towards_teacher():
  t_cfg = tiny_config("llama3-8b", ["init_weights_seed=1"])
  s_cfg = tiny_config("llama3-8b", ["init_weights_seed=2", "learning_rate=3e-3", "distill_alpha=0.0"])
  teacher, student = make_engine(t_cfg), make_engine(s_cfg)
  batch = {"inputs": torch.randint(0, 256, (2, 32)).int(), "targets": torch.randint(0, 256, (2, 32)).int()}
  losses = [float(T.distill_step(student, teacher, batch)["learning/loss"]) for _ in range(6)]
  assert losses[-1] < losses[0]


def test_gspo_token_weights_equal_autograd_and_trainer_runs():
  torch.manual_seed(2)
  N, S = 4, 6
  old = torch.randn(N, S)
  new = (old + 0.3 * torch.randn(N, S)).requires_grad_(True)
  adv = O.grpo_advantages(torch.tensor([1.0, 0.0, 3.0, 2.0]), 2)
  mask = torch.ones(N, S)
  mask[1, 4:] = 0
  # GSPO-token: s_it = sg[s_i] * pi_t / sg[pi_t], with s_i the length-normalised sequence ratio
  logr = (old - new) * mask
  s_i = torch.exp(logr.sum(1) / mask.sum(1))[:, None]
  s_it = s_i.detach() * torch.exp((old - new) - (old - new).detach())
  sur = -(torch.minimum(s_it * adv[:, None], s_it.clamp(0.8, 1.2) * adv[:, None]) * mask).sum() / mask.sum()
  sur.backward()
  val, w = O.gspo_weights(new.detach(), old, adv, mask, 0.2)
  assert torch.allclose(new.grad * mask.sum(), w, atol=1e-5) and abs(float(val) - float(sur)) < 1e-6
  cfg = tiny_config("llama3-8b", ["learning_rate=5e-3", "vocab_size=32", "max_prefill_predict_length=8"])
  tr = T.GRPOTrainer(make_engine(cfg), lambda p, c: float(c[0] % 2 == 0), group_size=2, max_new_tokens=3, loss_algo="gspo-token")
  m = tr.step([[1, 2, 3]])
  assert torch.isfinite(torch.as_tensor(m["learning/loss"]))


def test_use_dpo_through_the_train_cli(tmp_path):
  import json
  from helpers import TINY, BASE_YML
  from maxtext_b200.train import train as TR
  p = tmp_path / "pref.jsonl"
  p.write_text("\n".join(json.dumps({"prompt": f"q{i} ", "chosen": "yes yes", "rejected": "no no no"}) for i in range(8)))
  args = [a for a in TINY if not a.startswith(("steps", "dataset_type", "learning_rate=", "vocab_size", "per_device_batch_size"))] + [
      "model_name=llama3-8b", "steps=6", "use_dpo=true", "dataset_type=hf", f"hf_train_files={p}", "tokenizer_type=byte", "vocab_size=260",
      "per_device_batch_size=4", "learning_rate=5e-3", f"base_output_directory={tmp_path}", "run_name=dpo"]
  _, hist = TR.main(["train", BASE_YML] + args)
  acc = [float(h["dpo/reward_accuracy"]) for h in hist]
  loss = [float(h["dpo/loss"]) for h in hist]
  assert loss[-1] < loss[0] and acc[-1] >= acc[0] and abs(loss[0] - 0.6931) < 1e-3        # starts at log 2: policy = reference


def test_distillation_weight_schedules():
  import math
  from maxtext_b200.trainers.post_train.trainers import scheduled
  assert scheduled(5, 10, 0.5, None, "linear") == 0.5
  assert scheduled(5, 10, 0.5, 0.1, "constant") == 0.5
  assert abs(scheduled(5, 10, 0.5, 0.1, "linear") - 0.3) < 1e-9
  assert abs(scheduled(20, 10, 0.5, 0.1, "linear") - 0.1) < 1e-9
  assert abs(scheduled(5, 10, 2.0, 1.0, "cosine") - 1.5) < 1e-9 and abs(scheduled(0, 10, 2.0, 1.0, "cosine") - 2.0) < 1e-9
  import pytest
  with pytest.raises(ValueError):
    scheduled(1, 10, 1.0, 0.0, "step")
