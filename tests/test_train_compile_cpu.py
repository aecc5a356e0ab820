"""Ahead-of-time planner and estimator: no GPU, no process group, target worlds larger than this machine."""
import json

from helpers import BASE_YML
from maxtext_b200.config import pyconfig
from maxtext_b200.train import train_compile
from maxtext_b200.utils import estimator

ARGS = ["t", BASE_YML, "model_name=llama3-8b", "max_target_length=8192", "log_config=false"]


def test_plan_llama3_8b_fsdp8():
  cfg = pyconfig.initialize(ARGS + ["ici_fsdp_parallelism=8", "per_device_batch_size=2", "remat_policy=full"], num_devices=8)
  p = train_compile.plan(cfg, 8)
  assert p["parameters_total"] == 8030261248
  assert abs(p["parameters_per_rank"] - p["parameters_total"] / 8) / p["parameters_total"] < 1e-3
  assert p["fits"] and 20 < p["memory_total_gb"] < 80
  # ZeRO-3 traffic: two bf16 gathers and one fp32 reduce-scatter of 7/8 of the sharded parameters
  assert abs(p["per_step"]["all_gather_bytes"] - 2 * 2 * 8.03e9 * 7 / 8) / 2.8e10 < 0.02
  assert p["per_step"]["executed_tflops_per_device"] > p["per_step"]["model_tflops_per_device"]


def test_plan_reports_oom_and_more_shards_fit():
  big = ["model_name=llama3-70b", "per_device_batch_size=1", "max_target_length=8192", "log_config=false"]
  one = pyconfig.initialize(["t", BASE_YML] + big, num_devices=1)
  assert not train_compile.plan(one, 1)["fits"]
  many = pyconfig.initialize(["t", BASE_YML] + big + ["ici_fsdp_parallelism=16"], num_devices=16)
  assert train_compile.plan(many, 16)["fits"]


def test_cli_writes_plan(tmp_path, capsys):
  out = tmp_path / "plan.json"
  rc = train_compile.main(ARGS + ["compile_topology=b200-4", "ici_fsdp_parallelism=4", "per_device_batch_size=1", f"compiled_trainstep_file={out}"])
  assert rc == 0
  p = json.loads(out.read_text())
  assert p["world"] == 4 and p["units"][0]["name"] == "embed"


def test_estimator_prefers_less_recompute_when_it_fits():
  rows = estimator.search(ARGS + ["ici_fsdp_parallelism=8"], 8, batches=(1, 2, 4), policies=("minimal", "full"))
  assert rows and rows[0]["remat_policy"] == "minimal"
  full = [r for r in rows if r["remat_policy"] == "full"][0]
  assert full["per_device_batch_size"] >= rows[0]["per_device_batch_size"]


def test_every_recipe_resolves_and_plans():
  """Each named recipe parses into a valid configuration for its GPU count and yields a plan; the ones meant for one
  node fit 180 GB per GPU."""
  from maxtext_b200.benchmarks import benchmark_runner, recipes
  for r in recipes.RECIPES.values():
    cfg = pyconfig.initialize(["t", BASE_YML] + r.overrides() + ["log_config=false"], num_devices=r.gpus)
    p = train_compile.plan(cfg, r.gpus)
    assert p["world"] == r.gpus and p["parameters_total"] > 1e9, r.name
    assert p["fits"], (r.name, p["memory_total_gb"])
    cmd = benchmark_runner.command(r)
    assert ("torch.distributed.run" in cmd) == (r.gpus > 1)
