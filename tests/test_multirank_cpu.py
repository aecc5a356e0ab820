"""Multi-rank runs on CPU (gloo): a sharded mesh must reproduce the single-process loss curve.

The analogue of the reference's virtual-device tests (XLA_FLAGS=--xla_force_host_platform_device_count,
tests/unit/ulysses_collective_test.py:42): real collectives, tiny shapes, dense single-process oracle."""
import json
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE = ["base_emb_dim=64", "base_num_query_heads=4", "base_num_kv_heads=2", "head_dim=16", "base_mlp_dim=128",
        "base_num_decoder_layers=2", "vocab_size=512", "max_target_length=32", "dataset_type=synthetic", "dtype=float32",
        "hardware=cpu", "enable_checkpointing=false", "weight_init=normal", "log_config=false", "steps=3", "learning_rate=1e-3",
        "warmup_steps_fraction=0.0"]


def _free_port():
  s = socket.socket()
  s.bind(("127.0.0.1", 0))
  p = s.getsockname()[1]
  s.close()
  return p


def _merge(*lists):
  d = {}
  for l in lists:
    for e in l:
      d[e.split("=")[0]] = e     # later entries win
  return list(d.values())


def _launch(world, argv, timeout=300):
  """Start `world` gloo ranks of `argv`; returns (return codes, logs). A fresh rendezvous port per call."""
  port = _free_port()
  procs = []
  for r in range(world):
    env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
               MAXTEXT_B200_QUIET="1", OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    procs.append(subprocess.Popen(argv, cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
  logs = []
  for p in procs:
    try:
      o, _ = p.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
      for q in procs:
        q.kill()
      o = b"timed out"
      p.communicate()
    logs.append(o.decode(errors="replace"))
  return [p.returncode for p in procs], logs


def _launch_with_retry(world, argv):
  """The rendezvous on a freshly picked local port can lose a race with another process once in a while: a launch whose
  ranks fail is repeated once on a new port; a real failure fails both times and is reported."""
  codes, logs = _launch(world, argv)
  rendezvous = ("Address already in use", "EADDRINUSE", "Connection refused", "Connection reset", "connect() timed out", "DistNetworkError",
                "failed to connect", "Socket Timeout")
  if any(c != 0 for c in codes) and any(pat in l for l in logs for pat in rendezvous):
    # only a lost race for the port is repeated: a run that got further may have left checkpoints behind, and repeating it
    # would resume from them and report different steps
    codes, logs = _launch(world, argv)
  for c, l in zip(codes, logs):
    assert c == 0, l[-3000:]
  return logs


def run_ranks(world, overrides, tmp_path, tag):
  out = os.path.join(tmp_path, f"{tag}.json")
  _launch_with_retry(world, [sys.executable, os.path.join(ROOT, "tests", "multirank_worker.py"), out] + _merge(BASE, overrides))
  return json.load(open(out))


def _close(a, b, tol):
  assert len(a) == len(b)
  for x, y in zip(a, b):
    assert abs(x - y) <= tol * max(1.0, abs(y)), (a, b)


@pytest.fixture(scope="module")
def single(tmp_path_factory):
  return run_ranks(1, ["per_device_batch_size=4"], str(tmp_path_factory.mktemp("single")), "single")


def test_fsdp2_matches_single(single, tmp_path):
  got = run_ranks(2, ["per_device_batch_size=2", "ici_fsdp_parallelism=2"], str(tmp_path), "fsdp2")
  _close(got["loss"], single["loss"], 2e-4)
  _close(got["grad_norm"], single["grad_norm"], 2e-3)


def test_dp2_matches_single(single, tmp_path):
  got = run_ranks(2, ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_data_parallelism=2"], str(tmp_path), "dp2")
  _close(got["loss"], single["loss"], 2e-4)
  _close(got["grad_norm"], single["grad_norm"], 2e-3)


def test_fsdp2_x_tp2_matches_single(single, tmp_path):
  got = run_ranks(4, ["per_device_batch_size=1", "ici_fsdp_parallelism=2", "ici_tensor_parallelism=2"], str(tmp_path), "fsdp2tp2")
  _close(got["loss"], single["loss"], 2e-4)


def test_grad_accum_matches_single(single, tmp_path):
  got = run_ranks(1, ["per_device_batch_size=2", "gradient_accumulation_steps=2"], str(tmp_path), "ga2")
  _close(got["loss"], single["loss"], 2e-4)


def _diloco_oracle(overrides, replicas, steps, period, lr, mu):
  """Replica 0's loss curve from a hand-written simulation: independent engines, plain-tensor outer step."""
  import torch
  from maxtext_b200.config import pyconfig
  from maxtext_b200.input_pipeline import interface
  from maxtext_b200.train.engine import TrainEngine
  cfg = pyconfig.initialize(["w", os.path.join(ROOT, "maxtext_b200/configs/base.yml")] + _merge(BASE, overrides, [f"ici_diloco_parallelism={replicas}"]),
                            num_devices=replicas)     # same global batch as the multi-rank run; the engines below are single-rank
  engs = [TrainEngine(cfg, None, torch.device("cpu")) for _ in range(replicas)]
  its = [interface.create_data_iterator(cfg, r, replicas) for r in range(replicas)]
  outer = engs[0].store.master.clone()
  trace = torch.zeros_like(outer)
  losses = []
  for s in range(1, steps + 1):
    ms = [e.train_step(next(it)) for e, it in zip(engs, its)]
    losses.append(float(ms[0]["learning/loss"]))
    if s % period == 0:
      g = sum(outer - e.store.master for e in engs) / replicas
      trace = g + mu * trace
      outer = outer - lr * (g + mu * trace)
      for e in engs:
        e.store.master.copy_(outer)
        e.store.sync_compute_from_master()
  return losses


def test_diloco2_matches_simulation(tmp_path):
  over = ["enable_diloco=true", "diloco_sync_period=2", "diloco_outer_lr=0.7",
          "diloco_outer_momentum=0.9", "steps=5", "per_device_batch_size=2"]
  got = run_ranks(2, over + ["ici_diloco_parallelism=2"], str(tmp_path), "diloco2")
  want = _diloco_oracle(over, 2, 5, 2, 0.7, 0.9)
  assert got["loss"] == pytest.approx(want, rel=2e-5), (got["loss"], want)


@pytest.mark.parametrize("strategy", ["all_gather", "ulysses", "ring"])
def test_context_parallel2_matches_single(single, tmp_path, strategy):
  got = run_ranks(2, ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_context_parallelism=2",
                      f"context_parallel_strategy={strategy}"], str(tmp_path), f"cp2{strategy}")
  _close(got["loss"], single["loss"], 2e-4)
  _close(got["grad_norm"], single["grad_norm"], 2e-3)


def test_context_parallel_without_load_balance(single, tmp_path):
  got = run_ranks(2, ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_context_parallelism=2", "context_parallel_strategy=ulysses",
                      "context_parallel_load_balance=false"], str(tmp_path), "cp2nolb")
  _close(got["loss"], single["loss"], 2e-4)


def test_usp_ring2_x_ulysses2_matches_single(single, tmp_path):
  got = run_ranks(4, ["per_device_batch_size=1", "ici_fsdp_parallelism=1", "ici_context_parallelism=2", "ici_context_usp_ulysses_parallelism=2",
                      "context_parallel_strategy=usp"], str(tmp_path), "usp4")
  _close(got["loss"], single["loss"], 2e-4)
  _close(got["grad_norm"], single["grad_norm"], 2e-3)


def test_pipeline2_gpipe_matches_single(single, tmp_path):
  got = run_ranks(2, ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_pipeline_parallelism=2"], str(tmp_path), "pp2")
  _close(got["loss"], single["loss"], 2e-4)
  _close(got["grad_norm"], single["grad_norm"], 2e-3)


def test_pipeline2_circular_and_microbatches(tmp_path):
  four = ["base_num_decoder_layers=4"]
  ref = run_ranks(1, four + ["per_device_batch_size=4"], str(tmp_path), "single4")
  got = run_ranks(2, four + ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_pipeline_parallelism=2", "num_layers_per_pipeline_stage=1",
                             "num_pipeline_microbatches=4"], str(tmp_path), "pp2circ")
  _close(got["loss"], ref["loss"], 2e-4)
  _close(got["grad_norm"], ref["grad_norm"], 2e-3)


def test_pipeline2_x_fsdp2_matches_single(single, tmp_path):
  got = run_ranks(4, ["per_device_batch_size=1", "ici_fsdp_parallelism=2", "ici_pipeline_parallelism=2"], str(tmp_path), "pp2fsdp2")
  _close(got["loss"], single["loss"], 2e-4)
  _close(got["grad_norm"], single["grad_norm"], 2e-3)


def test_zero1_optimizer_sharded_over_data_matches_single(single, tmp_path):
  got = run_ranks(2, ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_data_parallelism=2", "shard_optimizer_over_data=true"],
                  str(tmp_path), "zero1")
  _close(got["loss"], single["loss"], 2e-4)
  _close(got["grad_norm"], single["grad_norm"], 2e-3)


def test_expert_parallel2_matches_single(tmp_path):
  moe = ["model_name=mixtral-8x7b", "override_model_config=true", "num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=64"]
  ref = run_ranks(1, moe + ["per_device_batch_size=4"], str(tmp_path), "moe1")
  got = run_ranks(2, moe + ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_expert_parallelism=2"], str(tmp_path), "ep2")
  _close(got["loss"], ref["loss"], 5e-4)


def test_ring_of_experts_matches_single(tmp_path):
  moe = ["model_name=mixtral-8x7b", "override_model_config=true", "num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=64"]
  ref = run_ranks(1, moe + ["per_device_batch_size=4"], str(tmp_path), "moe1r")
  got = run_ranks(2, moe + ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_expert_parallelism=2", "use_ring_of_experts=true"],
                  str(tmp_path), "roe2")
  _close(got["loss"], ref["loss"], 5e-4)
  _close(got["grad_norm"], ref["grad_norm"], 5e-3)


def _run_cli(world, overrides):
  """`python -m maxtext_b200.train.train` on `world` gloo ranks; returns rank 0's per-step losses."""
  import re
  logs = _launch_with_retry(world, [sys.executable, "-m", "maxtext_b200.train.train", os.path.join(ROOT, "maxtext_b200/configs/base.yml")]
                            + _merge(BASE, overrides))
  return [float(x) for x in re.findall(r"completed step: \d+.*?loss: ([0-9.]+)", logs[0])]


@pytest.mark.parametrize("layout", ["pp2", "fsdp2", "fsdp2tp2"])
def test_checkpoint_resume_reproduces_uninterrupted_run(tmp_path, layout):
  """Save under a sharded layout, stop, resume: the remaining steps equal those of a run that never stopped. Under pipeline
  parallelism every stage writes the layers it owns into the one shared tree; replicated tensors have exactly one writer."""
  par = {"pp2": (2, ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_pipeline_parallelism=2"]),
         "fsdp2": (2, ["per_device_batch_size=2", "ici_fsdp_parallelism=2"]),
         "fsdp2tp2": (4, ["per_device_batch_size=1", "ici_fsdp_parallelism=2", "ici_tensor_parallelism=2"])}[layout]
  world, over = par
  common = over + ["learning_rate_schedule_steps=6", f"base_output_directory={tmp_path}", "async_checkpointing=false"]
  full = _run_cli(world, common + ["steps=6", "run_name=full", "enable_checkpointing=false"])
  first = _run_cli(world, common + ["steps=4", "run_name=res", "enable_checkpointing=true", "checkpoint_period=2"])
  rest = _run_cli(world, common + ["steps=6", "run_name=res", "enable_checkpointing=true", "checkpoint_period=2"])
  assert first == full[:4] and len(rest) == 2, (full, first, rest)
  _close(rest, full[4:], 2e-4)


@pytest.mark.parametrize("packing", ["true", "false"])
def test_file_pipeline_resume_on_two_data_ranks_continues_the_same_batches(tmp_path, packing):
  """Both data-parallel ranks save their own reader position; after a stop at step 3 the remaining steps see the batches an
  uninterrupted run sees (equal losses), with and without packing windows."""
  data = tmp_path / "d.jsonl"
  with open(data, "w") as fh:
    for i in range(600):
      fh.write(json.dumps({"text": f"document {i} " + "abcdefg"[: i % 7] * (1 + i % 5)}) + "\n")
  common = ["per_device_batch_size=2", "ici_fsdp_parallelism=2", "dataset_type=hf", f"hf_train_files={data}", f"packing={packing}",
            "tokenizer_type=byte", "learning_rate_schedule_steps=6", f"base_output_directory={tmp_path}", "async_checkpointing=false",
            "checkpoint_period=3"]
  full = _run_cli(2, common + ["steps=6", "run_name=full", "enable_checkpointing=false"])
  first = _run_cli(2, common + ["steps=4", "run_name=res", "enable_checkpointing=true"])
  rest = _run_cli(2, common + ["steps=6", "run_name=res", "enable_checkpointing=true"])
  assert first == full[:4] and len(rest) == 2, (full, first, rest)
  assert len(set(full)) == len(full)           # different batches every step, so a replayed batch would show
  _close(rest, full[4:], 2e-4)
  assert sorted(os.listdir(tmp_path / "res" / "checkpoints" / "3" / "iter")) == ["process_0.json", "process_1.json"]


@pytest.mark.parametrize("model", ["llama3-8b", "qwen3-8b"])
def test_tp2_matches_single_including_grad_norm(tmp_path, model):
  """Pure tensor parallelism: the same tokens are scored on both ranks (count them once), per-head q/k norm scales see
  only the local heads (their gradients are summed over the tensor ranks), and replicated tensors enter the global
  gradient norm once. A wrong norm changes the clipping factor, so the curves are compared at a large learning rate."""
  q = [f"model_name={model}", "override_model_config=true", "steps=4", "learning_rate=1e-2"]
  one = run_ranks(1, q + ["per_device_batch_size=4"], str(tmp_path), "one")
  two = run_ranks(2, q + ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_tensor_parallelism=2"], str(tmp_path), "tp2")
  _close(two["loss"], one["loss"], 2e-5)
  _close(two["grad_norm"], one["grad_norm"], 2e-4)


@pytest.fixture(scope="module")
def moe_single(tmp_path_factory):
  return run_ranks(1, MOE_HOT + ["per_device_batch_size=4"], str(tmp_path_factory.mktemp("moe_single")), "single")


MOE_HOT = ["model_name=mixtral-8x7b", "override_model_config=true", "num_experts=4", "base_moe_mlp_dim=64", "load_balance_loss_weight=0.01",
           "steps=4", "learning_rate=1e-2"]


@pytest.mark.parametrize("layout", ["fsdp2", "ep2", "tp2", "ep2tp2"])
def test_moe_layouts_match_single_including_grad_norm(moe_single, tmp_path, layout):
  """Routed experts with the load-balance loss under FSDP, EP, TP and EP x TP: the balance loss is a per-rank mean (seeded
  with 1 / data shards), expert outputs are partial sums over the tensor ranks in every path, the tokens' and combine
  weights' gradients are summed over them where the combine precedes the reduction, and tensors that share a unit with
  differently replicated ones (router next to attention kernels, norm scales next to experts) are reduced and normed each
  with their own multiplicity."""
  world, par = {"fsdp2": (2, ["per_device_batch_size=2", "ici_fsdp_parallelism=2"]),
                "ep2": (2, ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_expert_parallelism=2"]),
                "tp2": (2, ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_tensor_parallelism=2"]),
                "ep2tp2": (4, ["per_device_batch_size=1", "ici_fsdp_parallelism=1", "ici_expert_parallelism=2", "ici_tensor_parallelism=2"])}[layout]
  got = run_ranks(world, MOE_HOT + par, str(tmp_path), layout)
  _close(got["loss"], moe_single["loss"], 2e-5)
  _close(got["grad_norm"], moe_single["grad_norm"], 2e-4)


@pytest.mark.parametrize("case", ["llama", "qwen3", "gpt3", "moe", "fsdp2xsp2"])
def test_tensor_sequence_parallel_matches_single(tmp_path, case):
  """`ici_tensor_sequence_parallelism`: tensor parallelism whose residual stream, norms and recompute checkpoints are split
  along the sequence (all-gather into a block, reduce-scatter out of it). Norm scales and post-reduction biases then see
  a part of the tokens only, so their gradients are summed over the tensor ranks; routed experts run on the gathered tokens."""
  hot = ["steps=4", "learning_rate=1e-2"]
  base = {"llama": [], "fsdp2xsp2": [], "qwen3": ["model_name=qwen3-8b", "override_model_config=true"],
          "gpt3": ["model_name=gpt3-6b", "override_model_config=true", "trainable_position_size=32"],
          "moe": ["model_name=mixtral-8x7b", "override_model_config=true", "num_experts=4", "base_moe_mlp_dim=64",
                  "load_balance_loss_weight=0.01"]}[case]
  world, par = (4, ["per_device_batch_size=1", "ici_fsdp_parallelism=2", "ici_tensor_sequence_parallelism=2"]) if case == "fsdp2xsp2" else \
      (2, ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_tensor_sequence_parallelism=2"])
  one = run_ranks(1, base + hot + ["per_device_batch_size=4"], str(tmp_path), "one")
  got = run_ranks(world, base + hot + par, str(tmp_path), "sp")
  _close(got["loss"], one["loss"], 2e-5)
  _close(got["grad_norm"], one["grad_norm"], 2e-4)


@pytest.mark.parametrize("layout", ["pp2xtp2", "cp2xtp2", "moe_pp2", "moe_cp2"])
def test_combined_layouts_match_single_including_grad_norm(single, moe_single, tmp_path, layout):
  """Pipeline x tensor and context x tensor meshes, and the load-balance loss under pipeline parallelism (each stage adds the
  loss of its own layers, seeded per micro-batch) and under context parallelism (the per-sequence routing statistics are
  means over the whole sequence, of which a rank holds a part)."""
  hot = ["steps=4", "learning_rate=1e-2"]
  world, base, par = {
      "pp2xtp2": (4, [], ["per_device_batch_size=1", "ici_fsdp_parallelism=1", "ici_pipeline_parallelism=2", "ici_tensor_parallelism=2"]),
      "cp2xtp2": (4, [], ["per_device_batch_size=1", "ici_fsdp_parallelism=1", "ici_context_parallelism=2", "ici_tensor_parallelism=2",
                          "context_parallel_strategy=all_gather"]),
      "moe_pp2": (2, MOE_HOT, ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_pipeline_parallelism=2"]),
      "moe_cp2": (2, MOE_HOT, ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_context_parallelism=2",
                               "context_parallel_strategy=all_gather"])}[layout]
  want = moe_single if base else run_ranks(1, hot + ["per_device_batch_size=4"], str(tmp_path), "one")
  got = run_ranks(world, base + hot + par, str(tmp_path), layout)
  _close(got["loss"], want["loss"], 2e-5)
  _close(got["grad_norm"], want["grad_norm"], 2e-4)


@pytest.mark.parametrize("case", ["lora", "masks"])
def test_frozen_parameters_under_fsdp_match_single(tmp_path, case):
  """LoRA and `trainable_parameters_mask` / `adamw_mask` with flat sharded optimizer state: frozen ranges get zero gradient
  and no decay on every shard, trained ranges are decayed on the shard that owns them."""
  over = {"lora": ["lora={enable_lora: true, lora_rank: 4, lora_alpha: 8.0}"],
          "masks": ["trainable_parameters_mask=['.*mlp.*']", "adamw_mask=['.*wo.*']"]}[case] + ["steps=4", "learning_rate=1e-2"]
  one = run_ranks(1, over + ["per_device_batch_size=4"], str(tmp_path), "one")
  two = run_ranks(2, over + ["per_device_batch_size=2", "ici_fsdp_parallelism=2"], str(tmp_path), "two")
  _close(two["loss"], one["loss"], 2e-5)
  _close(two["grad_norm"], one["grad_norm"], 2e-4)


def test_checkpoint_written_under_one_layout_resumes_under_another(tmp_path):
  """Resharding on restore: a run saved by 2 FSDP ranks continues on 2 tensor-parallel ranks and on a single rank, and the
  remaining steps equal those of an uninterrupted single-rank run (the tree on disk does not depend on the mesh)."""
  common = ["learning_rate_schedule_steps=6", f"base_output_directory={tmp_path}", "async_checkpointing=false"]
  full = _run_cli(1, common + ["per_device_batch_size=4", "steps=6", "run_name=full", "enable_checkpointing=false"])
  ck = ["enable_checkpointing=true", "checkpoint_period=2"]
  first = _run_cli(2, common + ck + ["per_device_batch_size=2", "ici_fsdp_parallelism=2", "steps=4", "run_name=a"])
  _close(first, full[:4], 2e-5)
  import shutil
  shutil.copytree(os.path.join(tmp_path, "a"), os.path.join(tmp_path, "b"))
  rest_tp = _run_cli(2, common + ck + ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_tensor_parallelism=2", "steps=6", "run_name=a"])
  rest_one = _run_cli(1, common + ck + ["per_device_batch_size=4", "steps=6", "run_name=b"])
  assert len(rest_tp) == 2 and len(rest_one) == 2
  _close(rest_tp, full[4:], 2e-4)
  _close(rest_one, full[4:], 2e-4)


@pytest.mark.parametrize("layout", ["tp2", "fsdp2xtp2"])
def test_lora_adapters_under_tensor_parallelism_match_single(tmp_path, layout):
  """Adapters follow their weight's split (column: B split, row: A split); the whole factor's gradient is summed over the
  tensor ranks, also when the unit is sharded over fsdp as well."""
  lora = ["lora={enable_lora: true, lora_rank: 4, lora_alpha: 8.0}", "weight_init=normal", "learning_rate=1e-2"]
  one = run_ranks(1, lora + ["per_device_batch_size=4"], str(tmp_path), "one")
  # the global batch is per_device_batch_size x ranks, whatever the ranks are used for
  world, par = (2, ["per_device_batch_size=2", "ici_fsdp_parallelism=1", "ici_tensor_parallelism=2"]) if layout == "tp2" else \
      (4, ["per_device_batch_size=1", "ici_fsdp_parallelism=2", "ici_tensor_parallelism=2"])
  got = run_ranks(world, lora + par, str(tmp_path), layout)
  _close(got["loss"], one["loss"], 2e-4)
  _close(got["grad_norm"], one["grad_norm"], 2e-3)
  assert one["loss"][-1] < one["loss"][0]


def test_two_slices_data_parallel_over_dcn_and_fsdp_inside_match_single(single, tmp_path):
  """num_slices=2: the `data` axis spans the slices (dcn), fsdp stays inside a slice (ici). Ranks of one slice are contiguous, the
  gradient is reduce-scattered inside the slice and only the shards cross slices."""
  from maxtext_b200.config import pyconfig
  from maxtext_b200.parallel.mesh import Mesh
  over = ["per_device_batch_size=1", "num_slices=2", "dcn_data_parallelism=2", "ici_fsdp_parallelism=2"]
  cfg = pyconfig.initialize(["t", os.path.join(ROOT, "maxtext_b200/configs/base.yml")] + _merge(BASE, over), num_devices=4)
  assert dict(zip(cfg.mesh_axes, cfg.mesh_shape))["data"] == 2 and dict(zip(cfg.mesh_axes, cfg.mesh_shape))["fsdp"] == 2
  m = Mesh(list(cfg.mesh_axes), list(cfg.mesh_shape), rank=0, world=4)
  assert m.ranks_along(("fsdp",), 0) == [0, 1] and m.ranks_along(("fsdp",), 2) == [2, 3]      # a slice = consecutive ranks
  assert m.ranks_along(("data",), 0) == [0, 2]
  got = run_ranks(4, over, str(tmp_path), "dcn2")
  _close(got["loss"], single["loss"], 2e-4)
  _close(got["grad_norm"], single["grad_norm"], 2e-3)
