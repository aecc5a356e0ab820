"""Small operator tools: multi-host launcher command lines, weight comparison."""
import io
import subprocess
import sys

import torch


def test_multihost_runner_builds_one_command_per_host_and_stops_on_failure(tmp_path, capsys):
  from maxtext_b200.orchestration import multihost_runner as M
  cmds = M.host_commands(["n0", "n1"], 8, ["python", "-m", "maxtext.train", "cfg.yml", "run_name=a b"], "/repo", port=1234, env={"NCCL_DEBUG": "WARN"})
  assert len(cmds) == 2 and cmds[0][0] == "ssh" and cmds[1][-2] == "n1"
  r1 = cmds[1][-1]
  assert "NNODES=2" in r1 and "NODE_RANK=1" in r1 and "JAX_COORDINATOR_ADDRESS=n0" in r1 and "JAX_COORDINATOR_PORT=1234" in r1
  assert "GPUS_PER_NODE=8" in r1 and "NCCL_DEBUG=WARN" in r1 and "gpu_multi_process_run.sh" in r1 and "'run_name=a b'" in r1
  assert M.main(["--hosts", "a,b,c", "--dry-run", "--", "echo", "hi"]) == 0
  assert capsys.readouterr().out.count("ssh ") == 3
  # run(): local stand-ins for ssh; host "bad" fails, the job's exit code is its code and output lines carry the host name
  def fake(argv, **kw):
    host = argv[-2]
    code = "import sys,time; print('up'); sys.stdout.flush(); " + ("sys.exit(3)" if host == "bad" else "time.sleep(30)")
    return subprocess.Popen([sys.executable, "-c", code], **kw)
  sink = io.StringIO()
  rc = M.run(["good", "bad"], 1, ["true"], "/repo", runner=fake, sink=sink)
  assert rc == 3 and "[good] up" in sink.getvalue() and "[bad] exited with 3" in sink.getvalue()


def test_weight_inspector_reports_structure_and_value_differences(tmp_path):
  from safetensors.torch import save_file
  from maxtext_b200.utils import weight_inspector as W
  a = {"layers.0.w": torch.ones(4, 4), "layers.1.w": torch.arange(6.0).view(2, 3), "only_a": torch.zeros(2)}
  b = {"layers.0.w": torch.ones(4, 4) + 1e-7, "layers.1.w": torch.arange(6.0).view(2, 3).clone(), "only_b": torch.zeros(2)}
  b["layers.1.w"][1, 2] = 9.0
  save_file(a, str(tmp_path / "a.safetensors"))
  torch.save(b, str(tmp_path / "b.pt"))
  rep = W.compare(W.load_weights(str(tmp_path / "a.safetensors")), W.load_weights(str(tmp_path / "b.pt")))
  assert rep["only_lhs"] == ["only_a"] and rep["only_rhs"] == ["only_b"] and rep["equal"] == 1 and not rep["match"]
  d = rep["different"][0]
  assert d["key"] == "layers.1.w" and d["max_abs"] == 4.0 and d["at"] == 5 and abs(d["fraction"] - 1 / 6) < 1e-6
  assert W.compare(a, b, pattern=r"layers\\.0")["match"]
  assert W.compare({"x": torch.zeros(2, 3)}, {"x": torch.zeros(3, 2)})["shape_mismatch"][0]["lhs"] == [2, 3]
  assert W.main(["--lhs", str(tmp_path / "a.safetensors"), "--rhs", str(tmp_path / "a.safetensors")]) == 0


def test_distillation_data_generation_filters_long_prompts_and_repeats_generations(tmp_path):
  import json
  from maxtext_b200.trainers.post_train.distillation import generate_distillation_data as G
  rows = [{"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "old answer"}]},
          {"messages": [{"role": "user", "content": "x" * 500}]},
          {"messages": [{"role": "assistant", "content": "orphan"}]},
          {"prompt": "plain"}]
  calls = []

  def teacher(prompts, max_new):
    calls.append(list(prompts))
    return [f"answer{len(calls)} to {p[-12:]!r}" for p in prompts]
  out = list(G.generate(rows, teacher, len, 100, column="messages", num_generations=2, batch_size=8))
  assert len(out) == 2 and len(calls) == 2 and G.generate.skipped == 3          # the long one, the orphan, and the row without `messages`
  assert out[0]["messages"][-1] == {"role": "assistant", "content": out[0]["completion"]} and len(out[0]["messages"]) == 2
  assert out[0]["prompt"].endswith("assistant: ") and out[0]["generation"] == 0 and out[1]["generation"] == 1
  plain = list(G.generate(rows, teacher, len, 100, column="prompt"))
  assert len(plain) == 1 and plain[0]["prompt"] == "plain" and "messages" not in plain[0]
  f = tmp_path / "p.jsonl"
  f.write_text("\n".join(json.dumps(r) for r in rows))
  assert G.read_rows(str(f)) == rows


def test_mxfp4_and_fp8_block_checkpoints_dequantize(tmp_path):
  import json
  from safetensors.torch import load_file, save_file
  from maxtext_b200.checkpoint_conversion import dequantize as D
  # every code decodes to its table value, low nibble first, scaled by 2^(s - 127)
  blocks = torch.tensor([[[0x21, 0xF7] + [0] * 14]], dtype=torch.uint8)              # codes 1, 2, 7, 15
  out = D.dequantize_mxfp4(blocks, torch.tensor([[128]], dtype=torch.uint8), torch.float32)
  assert out.shape == (1, 32) and out[0, :4].tolist() == [1.0, 2.0, 12.0, -12.0] and float(out[0, 4:].abs().sum()) == 0.0
  torch.manual_seed(0)
  w = torch.randn(3, 4, 64) * 0.3
  b, s = D.quantize_mxfp4(w)
  assert b.shape == (3, 4, 2, 16) and s.shape == (3, 4, 2)
  back = D.dequantize_mxfp4(b, s, torch.float32)
  scale = torch.exp2(s.float() - 127).repeat_interleave(32, -1)
  assert float(((back - w).abs() / scale).max()) <= 1.0 + 1e-6                        # within half the widest gap (2) of the grid
  assert torch.equal(D.dequantize_mxfp4(*D.quantize_mxfp4(back), torch.float32), back)  # grid values are fixed points
  # fp8 block scaling: ragged 200 x 300 weight with 2 x 3 tile scales
  wf = torch.randn(200, 300)
  sc = torch.rand(2, 3) + 0.5
  q = (wf / sc.repeat_interleave(128, 0)[:200].repeat_interleave(128, 1)[:, :300]).to(torch.float8_e4m3fn)
  deq = D.dequantize_fp8_blocks(q, sc, torch.float32)
  assert float((deq - wf).abs().max()) < 0.13 * float(wf.abs().max())
  # a directory with both kinds, the scale of one weight in another shard
  src, dst = tmp_path / "in", tmp_path / "out"
  src.mkdir()
  save_file({"experts.gate_up_proj_blocks": b, "experts.gate_up_proj_scales": s, "a.weight": q, "norm.weight": torch.ones(4)}, str(src / "m-1.safetensors"))
  save_file({"a.weight_scale_inv": sc}, str(src / "m-2.safetensors"))
  (src / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": {}}))
  (src / "config.json").write_text("{}")
  rep = D.convert_directory(str(src), str(dst), torch.float32)
  assert rep == {"files": 2, "rewritten": 2}
  got = load_file(str(dst / "m-1.safetensors"))
  assert set(got) == {"experts.gate_up_proj", "a.weight", "norm.weight"} and torch.equal(got["experts.gate_up_proj"], back)
  assert torch.allclose(got["a.weight"], deq) and (dst / "config.json").exists()
  wm = json.loads((dst / "model.safetensors.index.json").read_text())["weight_map"]
  assert wm["experts.gate_up_proj"] == "m-1.safetensors" and "a.weight_scale_inv" not in wm


def test_reference_module_paths_resolve_to_this_repository():
  import importlib
  for name in ("maxtext.train", "maxtext.train_compile", "maxtext.inference.decode", "maxtext.inference.maxengine.maxengine_server",
               "maxtext.inference.inference_microbenchmark", "maxtext.inference.mlperf.offline_mode", "maxtext.checkpoint_conversion.to_maxtext",
               "maxtext.checkpoint_conversion.to_huggingface", "maxtext.utils.standalone_checkpointer", "maxtext.utils.get_flops",
               "maxtext.utils.layerwise_quantization", "maxtext.eval.runner.run", "maxtext.trainers.post_train.sft.train_sft",
               "maxtext.trainers.post_train.rl.train_rl", "maxtext.trainers.tokenizer.train_tokenizer"):
    assert callable(getattr(importlib.import_module(name), "main")), name
