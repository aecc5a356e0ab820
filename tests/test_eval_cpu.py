"""Evaluation framework: scorers, dataset field mapping, and the three task kinds end to end on a tiny model, in-process
and through the serving loop's HTTP app."""
import json

import pytest
import torch

from helpers import tiny_config
from maxtext_b200 import eval as ev


def test_rouge_and_exact_match():
  r = ev.rouge(["the cat sat on the mat"], ["the cat sat on the mat"])
  assert r["rouge1"] == pytest.approx(100) and r["rouge2"] == pytest.approx(100) and r["rougeL"] == pytest.approx(100)
  r = ev.rouge(["the cat sat"], ["the dog sat down"])
  # unigrams: 2 of 3 predicted, 2 of 4 reference -> F = 2 * (2/3) * (1/2) / (2/3 + 1/2); bigrams share nothing; LCS = 2
  assert r["rouge1"] == pytest.approx(100 * 2 * (2 / 3) * 0.5 / (2 / 3 + 0.5)) and r["rouge2"] == 0 and r["rougeL"] == pytest.approx(r["rouge1"])
  assert ev.exact_match(["Paris.", "Rome"], ["paris", "Milan"])["exact_match"] == 0.5
  assert ev.exact_match(["so the total is 1,234 apples"], ["... #### 1234"], numeric=True)["exact_match"] == 1.0


def test_dataset_field_mapping(tmp_path):
  p = tmp_path / "d.jsonl"
  p.write_text("\n".join(json.dumps(r) for r in [
      {"question": "2+2?", "choices": ["3", "4"], "answer": "B"},
      {"system_prompt": "be brief", "question": "capital of France?", "output": "Paris"},
      {"text": "just some text to score"}]))
  s = ev.load_dataset("jsonl", path=str(p))
  assert s[0].kind == "choice" and s[0].answer == 1 and s[1].kind == "generate" and s[1].prompt.startswith("be brief") and s[1].reference == "Paris"
  assert s[2].kind == "perplexity"
  assert len(ev.load_dataset("jsonl", path=str(p), num_samples=2)) == 2
  with pytest.raises(KeyError):
    ev.load_dataset("nope")


@pytest.fixture(scope="module")
def backend():
  from maxtext_b200.inference.maxengine import MaxEngine
  cfg = tiny_config("llama3-8b", ["max_prefill_predict_length=16", "max_target_length=32", "tokenizer_type=byte", "vocab_size=260"])
  eng = MaxEngine(cfg)
  eng.load_params()                                  # random weights: the scores must depend on the text
  return ev.LocalBackend(cfg, engine=eng, slots=2)


def test_three_task_kinds_in_process(backend, tmp_path):
  run = ev.EvalRunner(backend, max_new_tokens=4)
  gen = run.run(ev.load_dataset("synthetic_copy", num_samples=3))
  assert gen["task"] == "generate" and len(gen["records"]) == 3 and 0 <= gen["metrics"]["rougeL"] <= 100
  mc = run.run([ev.EvalSample("2+2 =", choices=["3", "4", "5"], answer=1, kind="choice"),
                ev.EvalSample("sky is", choices=["blue", "green"], answer=0, kind="choice")])
  assert mc["task"] == "choice" and 0 <= mc["metrics"]["accuracy"] <= 1 and len(mc["records"][0]["scores"]) == 3
  # the choice scores are true sequence log-likelihoods: they match a direct computation
  b = backend
  ids = b._ids("2+2 =") + b._ids(" 4", bos=False)
  lg = b.engine.model.forward(torch.tensor(ids)[None])[0].float()
  lp = torch.log_softmax(lg[:-1], -1).gather(1, torch.tensor(ids)[1:, None])[:, 0]
  n = len(b._ids(" 4", bos=False))
  assert mc["records"][0]["scores"][1] == pytest.approx(float(lp[-n:].sum()) / n, rel=1e-5)
  ppl = run.run([ev.EvalSample("some text to score here", kind="perplexity")])
  assert ppl["metrics"]["perplexity"] > 1 and ppl["metrics"]["tokens"] > 0
  from maxtext_b200.eval.runner import write_report
  path = write_report(gen, str(tmp_path), "t")
  assert json.load(open(path))["metrics"]["samples"] == 3 and len(open(tmp_path / "t_samples.jsonl").read().splitlines()) == 3


def test_server_backend_against_the_serving_app(backend):
  pytest.importorskip("fastapi")
  pytest.importorskip("aiohttp")
  import socket
  import threading
  import uvicorn
  from maxtext_b200.inference.maxengine_server import ServingLoop, create_app
  loop = ServingLoop(backend.c, engine=backend.engine, tokenizer=backend.tok)
  loop.start()
  s = socket.socket()
  s.bind(("127.0.0.1", 0))
  port = s.getsockname()[1]
  s.close()
  server = uvicorn.Server(uvicorn.Config(create_app(loop), host="127.0.0.1", port=port, log_level="error"))
  th = threading.Thread(target=server.run, daemon=True)
  th.start()
  try:
    import time
    for _ in range(100):
      if server.started:
        break
      time.sleep(0.05)
    res = ev.EvalRunner(ev.ServerBackend(f"http://127.0.0.1:{port}", concurrency=3), max_new_tokens=3).run(
        ev.load_dataset("synthetic_copy", num_samples=4), "exact_match")
    assert res["metrics"]["samples"] == 4 and len(res["records"]) == 4
  finally:
    server.should_exit = True
    th.join(timeout=10)
    loop.stop()


def test_harness_adapter_methods(backend):
  from maxtext_b200.eval.harness import MaxTextLM
  lm = MaxTextLM(backend, max_gen_toks=4)
  (ll, greedy), (ll2, _) = lm.loglikelihood([("2+2 =", " 4"), ("2+2 =", " 5")])
  want, n = backend.loglikelihood("2+2 =", " 4")
  assert ll == pytest.approx(want, rel=1e-5) and isinstance(greedy, bool) and ll != ll2
  assert lm.loglikelihood_rolling([("some text here",)])[0] < 0
  gen = lm.generate_until([("repeat: abc", {"until": ["\n"], "max_gen_toks": 3})])
  assert isinstance(gen[0], str) and "\n" not in gen[0]
