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
      "model_name=llama3-8b", "steps=6", "use_dpo=true", "packing=false", "dataset_type=hf", f"hf_train_files={p}", "tokenizer_type=byte", "vocab_size=260",
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


def test_hooked_loop_calls_callbacks_in_order_and_stops_at_target_eval_loss():
  """The shared post-training loop: data hooks feed batches, training hooks see start / step / eval / end in order, and
  the run ends early once the evaluation loss reaches `target_eval_loss`."""
  from helpers import batch_of, make_engine, tiny_config
  from maxtext_b200.trainers.post_train import hooks as H
  cfg = tiny_config(extra=["steps=6", "eval_interval=2", "eval_steps=1", "target_eval_loss=100.0", "learning_rate=1e-3"])
  eng = make_engine(cfg)
  calls = []

  class Spy(H.MetricTrainingHooks):
    def on_train_start(self, loop):
      calls.append("start")
      super().on_train_start(loop)

    def on_train_step_end(self, loop, step, metrics, step_time):
      calls.append(f"step{step}")
      super().on_train_step_end(loop, step, metrics, step_time)

    def on_eval_step_end(self, loop, loss_sum, weights):
      calls.append("eval")
      super().on_eval_step_end(loop, loss_sum, weights)

    def on_train_end(self, loop):
      calls.append("end")
      super().on_train_end(loop)

  class OneBatch:
    def __iter__(self):
      return self

    def __next__(self):
      return batch_of(cfg)
  data = H.DataHooks(cfg, train_iterator=OneBatch(), eval_iterator=OneBatch())

  def eval_fn(batch):
    m = eng.eval_step(batch)
    return float(m["evaluation/total_loss"]), float(m["evaluation/total_weights"])
  hooks = Spy(cfg, is_writer=False)
  done = H.run_with_hooks(cfg, eng, hooks, data, eval_fn)
  # the evaluation after step 1 meets the (generous) target, which ends the run
  assert calls == ["start", "step0", "step1", "eval", "end"] and done == 2
  step_rows = [m for _, m in hooks.history if "learning/loss" in m]
  assert step_rows[0]["learning/total_weights"] > 0 and step_rows[0]["learning/perplexity"] > 1.0
  assert any("eval/avg_perplexity" in m for _, m in hooks.history)


def _rl_cfg(tmp_path, extra=()):
  from helpers import tiny_config
  return tiny_config(extra=["max_target_length=64", "max_prefill_predict_length=40", "per_device_batch_size=2", "steps=2", "vocab_size=300",
                            "tokenizer_type=byte", "learning_rate=1e-3", "decode_sampling_temperature=1.0", "eval_interval=1", "eval_steps=2",
                            "reasoning_start_token=<r>", "reasoning_end_token=</r>", "solution_start_token=<a>", "solution_end_token=</a>",
                            "reward_exact_format_match=0.5", "reward_partial_format_match=0.25", "penalty_incorrect_format=-0.25",
                            "reward_exact_answer=3.0", "reward_white_space_format_match=1.5", "penalty_incorrect_answer=-1.0", *extra])


def test_reward_functions_and_answer_extraction(tmp_path):
  """Format rewards follow the tag structure; the answer reward accepts exact text, white-space variants and numerically
  equal forms (through the verification workers), and penalises wrong or missing answers."""
  from maxtext_b200.trainers.post_train.rl import math_verify_pool as mvp, rewards as R
  c = _rl_cfg(tmp_path)
  good = "<r>2+2 is 4</r><a>\\boxed{4}</a>"
  assert R.extract_answer(good, c) == "4" and R.extract_answer("<a> 7 </a>", c) == "7" and R.extract_answer("nothing", c) == R.FALLBACK_ANSWER
  assert R.extract_answer("<a>\\boxed{\\frac{1}{2}}</a>", c) == "\\frac{1}{2}"
  assert R.extract_hash_answer("so the total is 18\n#### 18") == "18"
  assert R.match_format_exactly([""], [good, "4"], c) == [0.5, 0.0]
  assert R.match_format_approximately([""], [good, "<a>4"], c) == [1.0, -0.25 * 3 + 0.25]
  comps = [good, "<r>x</r><a>4.0</a>", "<r>x</r><a>5</a>", "no tags at all", "<a>1/2</a>", "<a>50%</a>"]
  ans = ['["4"]', '["4"]', '["4"]', '["4"]', '["0.5"]', '["0.5"]']
  assert R.check_numbers([""] * 6, comps, c, answer=ans, question=[""] * 6) == [3.0, 3.0, -0.25, -1.0, 3.0, 3.0]
  assert mvp.are_equal("\\boxed{1,000}", "1000") and not mvp.are_equal("12", "21")
  # the pooled path: more items than the in-process short cut takes, verified in spawned workers
  items = [(i, ["\\boxed{%d}" % i], ["\\boxed{%d.0}" % (i if i % 2 else i + 1)]) for i in range(6)]
  assert mvp.math_verify_pool(items, [0.0] * 6, reward=2.0, timeout=60.0, num_procs=2) == [0.0, 2.0, 0.0, 2.0, 0.0, 2.0]
  fns = R.build_reward_fns(c)
  assert [f.__name__ for f in fns] == ["match_format_exactly", "match_format_approximately", "check_numbers"]
  assert R.total_reward(fns, [""], [good], c, answer=['["4"]'], question=[""]) == [0.5 + 1.0 + 3.0]


def test_rl_train_loop_rolls_out_scores_and_updates(tmp_path):
  """`train_rl` end to end on a tiny model: rollouts from the policy's own weights, rewards from a user function named in
  the config, GRPO updates with a KL term to the starting policy, and the greedy evaluation pass."""
  import json
  from maxtext_b200.trainers.post_train.rl import train_rl
  data = tmp_path / "q.jsonl"
  with open(data, "w") as fh:
    for i in range(6):
      fh.write(json.dumps({"question": f"What is {i} + 1?", "answer": f"it is #### {i + 1}"}) + "\n")
  user = tmp_path / "my_rewards.py"
  user.write_text("def length_reward(prompts, completions, config, **kw):\n  return [float(len(c) % 5) for c in completions]\n")
  cfg = _rl_cfg(tmp_path, [f"hf_train_files={data}", f"hf_eval_files={data}", f"reward_functions_path={user}", "reward_functions=length_reward"])
  cfg = cfg.replace(rl={"num_generations": 2, "num_iterations": 2, "grpo_beta": 0.05, "grpo_epsilon": 0.2, "loss_algo": "grpo"})
  rows = train_rl.load_questions(str(data))
  assert rows[2] == {"question": "What is 2 + 1?", "answer": '["3"]'}
  trainer, hist = train_rl.rl_train(cfg)
  assert len(hist) == 2 and all("rl/mean_reward" in h and "rl/kl" in h and "learning/loss" in h for h in hist)
  assert all(h["eval/num_questions"] == 2 and 0.0 <= h["eval/accuracy"] <= 1.0 for h in hist)
  assert hist[0]["rl/kl"] >= 0.0 and hist[0]["rl/completion_tokens"] >= 1.0
  assert not torch.equal(trainer.ref_master, trainer.eng.store.master)          # the policy moved away from its start


def test_distillation_online_offline_and_learn_to_init(tmp_path):
  """Teacher top-k logits are written in resumable shards; the student trains from them (KL over the top-k support) and
  from an online teacher; learn-to-init copies the teacher's matching tensors, picking teacher layers for the student's."""
  import json
  import os
  from helpers import batch_of, make_engine, tiny_config
  from maxtext_b200.trainers.post_train.distillation import save_top_k_teacher_logits as S, train_distill as D
  t_cfg = tiny_config(extra=["base_num_decoder_layers=4", "steps=5"])
  s_cfg = tiny_config(extra=["base_num_decoder_layers=2", "steps=3", "learning_rate=2e-3", "distill_alpha=0.3", "distill_temperature=2.0",
                             "distill_temperature_end=1.0", "distill_temperature_schedule=linear"])
  teacher = make_engine(t_cfg)

  class Batches:
    def __init__(self):
      self.n = 0

    def __iter__(self):
      return self

    def __next__(self):
      self.n += 1
      b = batch_of(t_cfg)
      return {k: (v + self.n) % t_cfg.vocab_size if k in ("inputs", "targets") else v for k, v in b.items()}
  out = str(tmp_path / "topk")
  man = S.generate_and_save(t_cfg, teacher, Batches(), top_k=8, output_dir=out, shard_batches=2, max_batches=3)
  assert man["shards"] == ["shard_00000.npz", "shard_00001.npz"] and man["batches_done"] == 3
  man = S.generate_and_save(t_cfg, teacher, Batches(), top_k=8, output_dir=out, shard_batches=2, max_batches=5)   # resumes after batch 3
  assert man["batches_done"] == 5 and len(man["shards"]) == 3 and len(os.listdir(out)) == 4
  it = S.TopKShardIterator(out, batch=int(s_cfg.global_batch_size_to_load))
  b0 = next(it)
  vals, idx = S.teacher_top_k(teacher, {"inputs": b0["inputs"]}, 8)
  assert torch.equal(idx.cpu(), b0["top_k_indices"]) and torch.allclose(vals.cpu(), b0["top_k_logits"].float(), atol=0.05, rtol=0.02)
  # offline: the student's loss on a fixed shard batch falls
  student = make_engine(s_cfg)

  class Fixed:
    def __iter__(self):
      return self

    def __next__(self):
      return b0
  _, hist = D.train_distill(s_cfg.replace(offline_data_dir=out), student=student, data_iterator=Fixed())
  assert len(hist) == 3 and hist[-1]["learning/loss"] < hist[0]["learning/loss"]
  assert hist[0]["distill/temperature"] == 2.0 and 1.0 < hist[1]["distill/temperature"] < 2.0
  # online teacher + learn-to-init: student layers 0, 1 take teacher layers 0, 3
  student2 = make_engine(s_cfg)
  n = D.init_student_from_teacher(student2, teacher, [0, 3])
  assert n > 0
  name_s, name_t = "layers_1/mlp/wo/kernel", "layers_3/mlp/wo/kernel"
  assert torch.equal(student2.store.full_master(student2.store.params[name_s]), teacher.store.full_master(teacher.store.params[name_t]))
  _, hist2 = D.train_distill(s_cfg, student=student2, teacher=teacher, data_iterator=Fixed())
  assert hist2[-1]["learning/loss"] < hist2[0]["learning/loss"]


def test_learn_to_init_maps_teacher_attention_into_a_narrower_student():
  """Effective kernels follow the published contraction; training only the maps lowers the student's loss; collapsing writes them."""
  import torch
  from helpers import batch_of, make_engine, tiny_config
  from maxtext_b200.trainers.post_train.distillation.learn_to_init import LearnToInit, effective_kernel
  torch.manual_seed(0)
  # the contraction, against explicit loops
  C, A, B = torch.randn(5, 3, 4), torch.randn(3, 2), torch.randn(4, 6)
  k = effective_kernel(C, A, B)
  want = torch.zeros(5, 2, 6)
  for b in range(5):
    want[b] = A.t() @ C[b] @ B
  assert torch.allclose(k, want, atol=1e-5)
  Co, Ao, Bo = torch.randn(3, 4, 5), torch.randn(3, 2), torch.randn(6, 4)
  ko = effective_kernel(Co, Ao, Bo, is_output=True)
  assert ko.shape == (2, 6, 5) and torch.allclose(ko[..., 1], Ao.t() @ Co[..., 1] @ Bo.t(), atol=1e-5)
  W = torch.randn(3, 4, 2, 6)
  assert torch.allclose(effective_kernel(C, W=W), torch.einsum("bxy,xyuv->buv", C, W))
  # a student with 2 query heads of width 8 initialised from a "teacher" with 4 heads of width 16
  cfg = tiny_config("llama3-8b", ["base_num_query_heads=2", "base_num_kv_heads=2", "head_dim=8", "steps=8", "gradient_clipping_threshold=0"])
  eng = make_engine(cfg)
  D = cfg.emb_dim
  teacher = {}
  for i in range(cfg.num_decoder_layers):
    for proj in ("query", "key", "value"):
      teacher[f"layers_{i}/self_attention/{proj}/kernel"] = torch.randn(D, 4, 16) * 0.05
    teacher[f"layers_{i}/self_attention/out/kernel"] = torch.randn(4, 16, D) * 0.05
  lti = LearnToInit(eng, teacher, lr=2e-2, layer_indices=[0])
  assert set(lti.maps) == {n for n in teacher if n.startswith("layers_0/")}            # layer 1 keeps its own weights
  name = "layers_0/self_attention/query/kernel"
  p = eng.store.params[name]
  assert torch.allclose(eng.store.full_master(p).float(), lti._internal(name, lti.kernel(name)), atol=1e-6)
  other = eng.store.full_master(eng.store.params["layers_0/mlp/wi_0/kernel"]).clone()
  batch = batch_of(cfg)
  losses = [lti.step(batch)["loss"] for _ in range(8)]
  assert losses[-1] < losses[0]
  assert torch.equal(eng.store.full_master(eng.store.params["layers_0/mlp/wi_0/kernel"]), other)   # only the maps moved
  final = lti.collapse()
  assert torch.allclose(eng.store.full_master(p).float(), lti._internal(name, final[name]), atol=1e-6)
  g = LearnToInit(make_engine(cfg), teacher, general_map=True, layer_indices=[1])
  assert g.maps["layers_1/self_attention/out/kernel"]["train"]["W"].shape == (4, 16, 2, 8)
  assert g.step(batch)["loss"] > 0
