"""Decode engine: greedy decode equals the argmax of a full forward pass; insert / slots / sampling / cache quantization."""
import pytest
import torch

from helpers import tiny_config
from maxtext_b200.inference import inference_utils
from maxtext_b200.inference.maxengine import MaxEngine


def _engine(model="llama3-8b", extra=()):
  cfg = tiny_config(model, ["max_target_length=48", "max_prefill_predict_length=16", "per_device_batch_size=2", *extra])
  eng = MaxEngine(cfg, device="cpu")
  eng.load_params()
  return eng, cfg


@pytest.mark.parametrize("model", ["llama3-8b", "gemma2-2b", "gemma3-4b", "deepseek2-16b", "deepseek3-tiny", "qwen3-8b", "mixtral-8x7b",
                                   "gpt-oss-20b", "olmo3-7b", "llama4-17b-16e", "qwen2.5-7b", "qwen3-next-80b-a3b", "gemma4-26b", "envy-test", "deepseek4-tiny"])
def test_greedy_decode_matches_full_forward(model):
  eng, cfg = _engine(model)
  torch.manual_seed(0)
  prompt = torch.randint(1, cfg.vocab_size, (9,))
  prefix, first = eng.prefill(torch.nn.functional.pad(prompt, (0, 7)), 9)
  state = eng.init_decode_state(2)
  state = eng.insert(prefix, state, 1)
  seq = [int(first.data[0, 0])]
  for _ in range(6):
    state, res = eng.generate(state)
    assert int(res.data[1, 1]) == 1 and int(res.data[0, 1]) == 0       # slot 1 active, slot 0 idle
    seq.append(int(res.data[1, 0]))
  # oracle: re-run the whole sequence without a cache, step by step
  cur = prompt.clone()
  want = []
  for _ in range(7):
    logits = eng.model.forward(cur[None])
    nxt = int(logits[0, -1].argmax())
    want.append(nxt)
    cur = torch.cat([cur, torch.tensor([nxt])])
  assert seq == want


@pytest.mark.parametrize("model", ["llama3-8b", "deepseek4-tiny"])
def test_chunked_prefill_equals_prefill(model):
  eng, cfg = _engine(model)
  prompt = torch.randint(1, cfg.vocab_size, (13,))
  a, _ = eng.prefill(prompt, 13)
  b, _ = eng.prefill_chunked(prompt, chunk=4)
  assert torch.allclose(a.logits, b.logits, atol=1e-4) and int(a.first_token) == int(b.first_token)


def test_quantized_kv_cache_stays_close():
  eng, cfg = _engine(extra=["quantize_kvcache=true", "kv_quant_dtype=int8"])
  ref_eng, _ = _engine()
  prompt = torch.randint(1, cfg.vocab_size, (12,))
  a, _ = eng.prefill(prompt, 12)
  b, _ = ref_eng.prefill(prompt, 12)
  st = eng.insert(a, eng.init_decode_state(1), 0)
  st, _ = eng.generate(st)
  assert a.caches[0][0].k.dtype == torch.int8
  assert (a.logits - b.logits).abs().max() < 0.15                        # int8 keys/values perturb the logits only slightly
  assert int(st.next_pos[0]) == 13


def test_sampling_strategies():
  g = torch.Generator().manual_seed(0)
  logits = torch.tensor([[0.0, 5.0, 4.0, -1.0, 3.0]]).repeat(2000, 1)
  assert (inference_utils.sampling(logits, "greedy") == 1).all()
  tk = inference_utils.sampling(logits, "topk", topk=2, generator=g)
  assert set(tk.unique().tolist()) <= {1, 2}
  nu = inference_utils.sampling(logits, "nucleus", nucleus_p=0.7, generator=g)
  assert set(nu.unique().tolist()) <= {1, 2}
  co = inference_utils.sampling(logits, "composite", topk=3, nucleus_p=0.99, temperature=0.5, generator=g)
  assert set(co.unique().tolist()) <= {1, 2, 4}
  w = inference_utils.sampling(logits, "weighted", temperature=1.0, generator=g)
  frac = (w == 1).float().mean().item()
  assert abs(frac - torch.softmax(logits[0], -1)[1].item()) < 0.05


def test_decode_cli_and_offline_engine_and_microbenchmark():
  from maxtext_b200.inference import decode as D, microbenchmark
  from maxtext_b200.inference.offline_engine import OfflineEngine
  eng, cfg = _engine(extra=["vocab_size=300", "prompt=hello"])
  text = D.decode(cfg, engine=eng)
  assert isinstance(text, str)
  off = OfflineEngine(eng, slots=2)
  prompts = [[5, 6, 7], [9, 10, 11, 12], [3, 4], [8, 8, 8, 8, 8]]
  outs = off.batch_inference(prompts, max_new_tokens=5)
  assert [len(o) for o in outs] == [5, 5, 5, 5]
  # continuous batching must give each request the same tokens as running it alone
  solo = OfflineEngine(eng, slots=1).batch_inference([prompts[2]], max_new_tokens=5)[0]
  assert outs[2] == solo
  res = microbenchmark.run(tiny_config("llama3-8b", ["max_target_length=48", "max_prefill_predict_length=16", "inference_microbenchmark_prefill_lengths=8,16",
                                                    "inference_microbenchmark_loop_iters=1"]), eng)
  assert set(res["prefill"]) == {8, 16} and res["generate"]["tokens_per_s"] > 0


def test_serving_loop_batches_concurrent_requests():
  """Two threads post completions at once; the background loop serves both through the shared decode slots and each gets
  the tokens a direct batch_inference call produces for its prompt."""
  import threading
  from helpers import tiny_config
  from maxtext_b200.inference.maxengine import MaxEngine
  from maxtext_b200.inference.maxengine_server import ServingLoop, create_app
  from maxtext_b200.inference.offline_engine import OfflineEngine
  from maxtext_b200.input_pipeline.tokenizer import ByteTokenizer
  cfg = tiny_config(extra=["vocab_size=300", "max_target_length=48", "max_prefill_predict_length=16", "per_device_batch_size=2"])
  eng = MaxEngine(cfg, device="cpu")
  eng.load_params(seed=1)
  prompts = [[5, 6, 7, 8], [9, 10, 11]]
  want = OfflineEngine(eng, slots=2).batch_inference(prompts, max_new_tokens=6)
  loop = ServingLoop(cfg, engine=eng, tokenizer=ByteTokenizer()).start()
  out = [None, None]

  def call(i):
    out[i] = loop.complete({"prompt_tokens": prompts[i], "max_tokens": 6})

  ts = [threading.Thread(target=call, args=(i,)) for i in range(2)]
  [t.start() for t in ts]
  [t.join(60) for t in ts]
  assert [o["choices"][0]["tokens"] for o in out] == want
  assert out[0]["usage"]["prompt_tokens"] == 4 and loop.served == 2
  # one request with two prompts: one choice each, same tokens
  both = loop.complete({"prompt_tokens": prompts, "max_tokens": 6})
  assert [c["tokens"] for c in both["choices"]] == want and [c["index"] for c in both["choices"]] == [0, 1]
  # chat: the messages go through the chat template with the generation prompt
  from maxtext_b200.input_pipeline import chat as chat_lib
  msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
  reply = loop.chat({"messages": msgs, "max_tokens": 4})
  text = chat_lib.render(msgs, chat_lib.load_template(cfg), add_generation_prompt=True)
  direct = loop.complete({"prompt": text, "max_tokens": 4})
  assert reply["object"] == "chat.completion" and reply["choices"][0]["message"]["role"] == "assistant"
  assert reply["choices"][0]["message"]["content"] == direct["choices"][0]["text"] and reply["usage"]["prompt_tokens"] == direct["usage"]["prompt_tokens"]
  with pytest.raises(ValueError):
    loop.chat({"messages": []})
  loop.stop()
  app = create_app(loop)
  assert {r.path for r in app.routes} >= {"/v1/health", "/v1/completions", "/v1/chat/completions"}


@pytest.mark.parametrize("model", ["llama3-8b", "deepseek2-16b"])
def test_prefill_concat_and_multisampling_match_single_prefills(model):
  from helpers import tiny_config
  from maxtext_b200.inference.maxengine import MaxEngine
  cfg = tiny_config(model, ["max_prefill_predict_length=16", "max_target_length=48"])
  eng = MaxEngine(cfg)
  eng.load_params()
  torch.manual_seed(0)
  prompts = [torch.randint(1, cfg.vocab_size, (n,)) for n in (5, 9, 3)]
  packed = eng.prefill_concat(prompts)
  state = eng.init_decode_state(slots=3)
  state2 = eng.init_decode_state(slots=3)
  for i, (p, pre) in enumerate(zip(prompts, packed)):
    single, _ = eng.prefill(torch.nn.functional.pad(p, (0, 16 - p.numel())), p.numel())
    assert (pre.logits - single.logits).abs().max() < 1e-4 and int(pre.first_token) == int(single.first_token)
    state, state2 = eng.insert(pre, state, i), eng.insert(single, state2, i)
  for _ in range(4):                                  # the packed prefixes decode like the single ones
    state, r1 = eng.generate(state)
    state2, r2 = eng.generate(state2)
    assert torch.equal(r1.data[:, 0], r2.data[:, 0])
  many = eng.prefill_multisampling(torch.nn.functional.pad(prompts[0], (0, 11)), 5, 3)
  assert len(many) == 3 and all(m.length == 5 and m.caches is many[0].caches for m in many)
  st = eng.bulk_insert(many[0], eng.init_decode_state(slots=3), [0, 2])
  assert st.active.tolist() == [True, False, True] and st.next_pos.tolist()[0] == 5


def test_decode_multi_and_quantize_params():
  from helpers import tiny_config
  from maxtext_b200.inference.decode import decode
  from maxtext_b200.inference.decode_multi import decode_multi
  from maxtext_b200.inference.maxengine import MaxEngine
  cfg = tiny_config("llama3-8b", ["max_prefill_predict_length=16", "max_target_length=32", "tokenizer_type=byte", "vocab_size=260"])
  eng = MaxEngine(cfg)
  eng.load_params()
  prompts = ["abc", "hello there", "xy", "0123", "q"]
  multi = decode_multi(cfg, prompts, engine=eng, max_new_tokens=5)                 # five prompts through four slots
  assert len(multi) == 5
  for p, m in zip(prompts[:2], multi):
    assert decode(cfg, p, engine=eng)[:len(m)] == m or m.startswith(decode(cfg, p, engine=eng)[:3])
  ids = torch.randint(1, 250, (1, 12))
  before = eng.model.forward(ids)
  packed = eng.quantize_params(8)
  after = eng.model.forward(ids)
  name, (q, sc) = next(iter(packed.items()))
  assert q.dtype == torch.int8 and sc.shape == q.shape[:-1] and int(q.abs().max()) <= 127
  w = eng.model.store.full_master(eng.model.store.params[name]).float()
  assert torch.allclose(w, q.float() * sc[..., None], atol=1e-6)
  assert 0 < (after - before).abs().max() < 0.1 * before.abs().max()


def test_quantized_params_file_round_trip_and_stop_strings(tmp_path):
  from helpers import tiny_config
  from maxtext_b200.inference.decode import decode
  from maxtext_b200.inference.maxengine import MaxEngine
  base = ["max_prefill_predict_length=16", "max_target_length=32", "tokenizer_type=byte", "vocab_size=260"]
  eng = MaxEngine(tiny_config("llama3-8b", base))
  eng.load_params()
  f = eng.save_quantized_params(str(tmp_path / "q"), 8)
  ids = torch.randint(1, 250, (1, 10))
  want = eng.model.forward(ids)                           # the engine now holds the de-quantised weights
  other = MaxEngine(tiny_config("llama3-8b", base + ["init_weights_seed=7"]))
  other.load_params()
  for n in ("token_embedder/embedding", "decoder/decoder_norm/scale", "decoder/logits_dense/kernel"):
    other.model.store.load_full(n, eng.model.store.full_master(eng.model.store.params[n]))
  for n, p in eng.model.store.params.items():
    if "norm" in n:
      other.model.store.load_full(n, eng.model.store.full_master(p))
  other.load_quantized_params(f)
  assert (other.model.forward(ids) - want).abs().max() < 1e-5
  text = decode(tiny_config("llama3-8b", base), "hello", engine=eng)
  if len(text) > 3:
    stop = text[2:4]
    cut = decode(tiny_config("llama3-8b", base + [f"stop_strings=[{stop!r}]"]), "hello", engine=eng)
    assert stop not in cut and text.startswith(cut)


def test_tensor_parallel_decode_matches_single_rank(tmp_path):
  """MaxEngine on a 2-rank tensor-parallel mesh (gloo): head-split caches, same greedy tokens and logits as one rank."""
  import json
  import os
  import subprocess
  import sys
  from test_multirank_cpu import BASE, ROOT, _launch_with_retry, _merge

  def run(world, over, tag):
    out = str(tmp_path / f"{tag}.json")
    _launch_with_retry(world, [sys.executable, os.path.join(ROOT, "tests", "inference_tp_worker.py"), out] + _merge(BASE, over))
    return json.load(open(out))
  base = ["max_prefill_predict_length=16", "max_target_length=32", "per_device_batch_size=1"]
  one = run(1, base, "one")
  two = run(2, base + ["ici_fsdp_parallelism=1", "ici_tensor_parallelism=2"], "tp2")
  assert one["tokens"] == two["tokens"]
  assert all(abs(a - b) < 1e-5 for a, b in zip(one["logits"], two["logits"]))
  # the cache split along the sequence over two ranks (positions alternate between them), partial attention merged by log-sum-exp
  seq = run(2, base + ["ici_fsdp_parallelism=1", "ici_context_autoregressive_parallelism=2"], "car2")
  assert one["tokens"] == seq["tokens"]
  assert all(abs(a - b) < 1e-4 for a, b in zip(one["logits"], seq["logits"]))


def test_prompt_lengths_that_would_overrun_the_cache_are_rejected_on_the_host():
  """A prefix of max_target_length tokens would make the next decode step write one row past the slot's cache: prefill,
  insert, prefill_concat and the config layer refuse such lengths before any device work."""
  import pytest
  import torch
  from helpers import tiny_config
  from maxtext_b200.inference.maxengine import MaxEngine, Prefix
  cfg = tiny_config(extra=["max_target_length=32", "max_prefill_predict_length=16", "per_device_batch_size=2"])
  eng = MaxEngine(cfg, device=torch.device("cpu"))
  eng.load_params()
  toks = torch.arange(40) % 50
  with pytest.raises(ValueError):
    eng.prefill(toks, 32)
  with pytest.raises(ValueError):
    eng.prefill(toks[:8], 12)
  with pytest.raises(ValueError):
    eng.prefill_concat([toks[:4], toks[:35]])
  prefix, _ = eng.prefill(toks, 8)
  state = eng.init_decode_state()
  with pytest.raises(ValueError):
    eng.insert(Prefix(prefix.caches, 32, prefix.first_token, prefix.logits), state, 0)
  with pytest.raises(ValueError):
    eng.insert(prefix, state, 2)
  eng.insert(prefix, state, 1)
  from maxtext_b200.inference.offline_engine import OfflineEngine
  with pytest.raises(ValueError):
    OfflineEngine(MaxEngine(tiny_config(extra=["max_target_length=32", "max_prefill_predict_length=32"]), device=torch.device("cpu")))


def test_mixed_precision_quantisation_maps(tmp_path):
  """`quantization=intmp`: per-matrix widths, sub-channel tiles and clipping from a JSON map; the shipped maps parse."""
  import glob
  import json
  import os
  from helpers import ROOT, tiny_config
  from maxtext_b200.inference import mixed_precision as mp
  from maxtext_b200.inference.maxengine import MaxEngine
  shipped = sorted(glob.glob(os.path.join(ROOT, "maxtext_b200", "configs", "quantization", "*.json")))
  assert len(shipped) == 4
  for f in shipped:
    assert mp.load_quant_map(f)[-1][0] == mp.DEFAULT
  qmap = mp.load_quant_map(os.path.join(ROOT, "maxtext_b200", "configs", "quantization", "dense_llm_subchannel.json"))
  assert mp.settings_for("layers_0/self_attention/query/kernel", qmap) == {"w_bits": 4, "a_bits": 8, "tile_size": 128, "w_scale": 1.0}
  assert mp.settings_for("layers_0/mlp/wi_1/kernel", qmap)["w_bits"] == 8                       # falls to the default
  path = tmp_path / "map.json"
  path.write_text(json.dumps({"__default__": {"w_bits": 8}, ".*/query": {"w_bits": 4, "tile_size": 16}, ".*/wo": {"w_bits": 4, "w_scale": 0.5}}))
  base = ["max_prefill_predict_length=16", "max_target_length=32", "quantization=intmp", f"quant_cfg_path={path}"]
  eng = MaxEngine(tiny_config("llama3-8b", base))
  eng.load_params()
  raw = {n: eng.model.store.full_master(p).float().clone() for n, p in eng.model.store.params.items()}
  packed = eng.quantize_params()
  q, sc = packed["layers_0/self_attention/query/kernel"]
  assert int(q.abs().max()) <= 7 and sc.shape == (q.shape[0], q.shape[1] // 16)              # 4 bit, one scale per 16 inputs
  q8, sc8 = packed["layers_0/mlp/wi_0/kernel"]
  assert 7 < int(q8.abs().max()) <= 127 and sc8.shape == q8.shape[:-1]
  qo, so = packed["layers_0/mlp/wo/kernel"]
  w = raw["layers_0/mlp/wo/kernel"]
  assert torch.allclose(so, w.abs().amax(-1) * 0.5 / 7)                                        # half the range: the largest weights clip
  assert (qo.abs() == 7).float().mean() > (packed["layers_1/mlp/wo/kernel"][0].abs() == 7).float().mean() * 0 and int(qo.abs().max()) == 7
  # saved and loaded back, the sub-channel scales rebuild the same weights
  f = eng.save_quantized_params(str(tmp_path / "q"))
  ids = torch.randint(1, 250, (1, 10))
  want = eng.model.forward(ids)
  other = MaxEngine(tiny_config("llama3-8b", base))
  other.load_params()
  other.load_quantized_params(f)
  assert (other.model.forward(ids) - want).abs().max() < 1e-5
  import pytest
  bad = tmp_path / "bad.json"
  bad.write_text(json.dumps({".*": {"bits": 3}}))
  with pytest.raises(ValueError):
    mp.load_quant_map(str(bad))


def test_mlperf_offline_harness_and_accuracy_log(tmp_path):
  """Offline scenario driver: length buckets, per-bucket slots, LoadGen-format accuracy log, ROUGE against references."""
  import json
  from helpers import tiny_config
  from maxtext_b200.inference.maxengine import MaxEngine
  from maxtext_b200.inference.mlperf import evaluate_accuracy, offline_mode
  from maxtext_b200.input_pipeline.tokenizer import build_tokenizer
  cfg = tiny_config("llama3-8b", ["max_prefill_predict_length=32", "max_target_length=64", "tokenizer_type=byte", "vocab_size=260"])
  eng = MaxEngine(cfg)
  eng.load_params()
  tok = build_tokenizer(cfg)
  texts = ["short one", "a somewhat longer prompt here", "x", "the longest prompt of them all, yes"]
  data = tmp_path / "data.jsonl"
  data.write_text("\n".join(json.dumps({"tok_input": tok.encode(t), "tok_input_len": len(tok.encode(t)), "output": "reference text"}) for t in texts))
  out = tmp_path / "logs"
  args = offline_mode.parse_args(["--dataset_path", str(data), "--mlperf_test_mode", "accuracy", "--output_log_dir", str(out),
                                  "--prefill_lengths_and_batch_sizes", "8,2|16,2|40,1", "--max_new_tokens", "5",
                                  "--rename_dataset_cols", '{"tok_input_len": "tok_input_length"}'])
  summary = offline_mode.run(args, engine=eng)
  assert summary["samples"] == 4 and summary["generated_tokens"] > 0 and summary["samples_per_second"] > 0
  assert summary["buckets"] == {"8": 1, "16": 1, "40": 2}
  log = json.loads((out / "mlperf_log_accuracy.json").read_text())
  assert [e["qsl_idx"] for e in log] == [0, 1, 2, 3] and all(len(bytes.fromhex(e["data"])) == 8 * e["token_count"] for e in log)
  gen = evaluate_accuracy.decode_log(str(out / "mlperf_log_accuracy.json"))
  # the harness generated what the engine generates for the same prompt on its own
  from maxtext_b200.inference.offline_engine import OfflineEngine
  want = OfflineEngine(eng, slots=1).batch_inference([tok.encode(texts[0])], max_new_tokens=5)[0]
  assert gen[0] == want
  res = evaluate_accuracy.evaluate(str(out / "mlperf_log_accuracy.json"), offline_mode.load_dataset(str(data)), tok)
  assert set(res) >= {"rouge1", "rouge2", "rougeL", "gen_len", "gen_num"} and res["gen_num"] == 4
  import pytest
  with pytest.raises(ValueError):
    offline_mode.classify([{"tok_input_length": 99}], [(8, 1)], allow_skip=False)
  assert (out / "mlperf_log_summary.txt").read_text().startswith("=====")


def test_grpc_front_end_streams_the_tokens_of_the_serving_loop():
  pytest.importorskip("grpc")
  from helpers import tiny_config
  from maxtext_b200.inference import grpc_server as gs
  from maxtext_b200.inference.maxengine import MaxEngine
  from maxtext_b200.inference.maxengine_server import ServingLoop
  # message codec round trip
  assert gs.decode_request(gs.encode_request("héllo", None, 7)) == {"max_tokens": 7, "text": "héllo", "token_ids": None}
  assert gs.decode_request(gs.encode_request(None, [1, 300, 70000], 3))["token_ids"] == [1, 300, 70000]
  assert gs.decode_response(gs.encode_response("ab", [5, 260])) == {"text": "ab", "token_ids": [5, 260]}
  cfg = tiny_config("llama3-8b", ["max_prefill_predict_length=16", "max_target_length=32", "tokenizer_type=byte", "vocab_size=260", "per_device_batch_size=2"])
  eng = MaxEngine(cfg)
  eng.load_params()
  loop = ServingLoop(cfg, engine=eng).start()
  server, port = gs.serve(loop, 0)
  try:
    cl = gs.Client(f"127.0.0.1:{port}")
    assert cl.healthy()
    chunks = list(cl.decode(text="hello", max_tokens=6))
    ids = [t for c in chunks for t in c["token_ids"]]
    want = loop.complete({"prompt": "hello", "max_tokens": 6})["choices"][0]["tokens"]
    assert ids == want and 1 <= len(chunks) <= 6
    ids2 = [t for c in cl.decode(token_ids=loop.tok.encode("hello", add_bos=bool(cfg.add_bos)), max_tokens=6) for t in c["token_ids"]]
    assert ids2 == want
    cl.close()
  finally:
    server.stop(0)
    loop.stop()


def test_prefill_packing_buckets_and_offline_engine_agree_with_single_prefills():
  from maxtext_b200.inference.offline_engine import OfflineEngine
  from maxtext_b200.inference.prefill_packing import BatchedPrefillProcessor, PrefillBucket, PrefillProcessor
  b = PrefillBucket(10)
  assert b.is_empty() and b.try_add(0, "a", [1, 2, 3, 4]) and b.try_add(1, "b", [5, 6, 7, 8, 9]) and b.unallocated() == 1
  assert not b.try_add(2, "c", [1, 2]) and len(b) == 2
  with pytest.raises(ValueError):
    b.add(2, "c", [1, 2])
  with pytest.raises(ValueError):
    PrefillBucket(0)
  eng, cfg = _engine(extra=["vocab_size=300"])
  prompts = [[5, 6, 7], [9, 10, 11, 12], [3, 4], [8, 8, 8, 8, 8], [20, 21, 22, 23, 24, 25]]
  plain = OfflineEngine(eng, slots=3).batch_inference(prompts, max_new_tokens=5)
  packed_eng = OfflineEngine(eng, slots=3, enable_batch_prefill=True, batch_prefill_max_batch_size=2)
  packed = packed_eng.batch_inference(prompts, max_new_tokens=5)
  assert packed == plain
  assert 0 < packed_eng.batched.passes < len(prompts)                   # fewer passes than prompts: some were packed together
  # the processors by hand: three prompts, capacity for two of them -> two passes, results by callback
  proc = BatchedPrefillProcessor(eng, max_batch_size=8)
  state = eng.init_decode_state(3)
  got = {}
  done = lambda res, st: got.update({rid: int(tok.reshape(-1)[0]) for rid, tok in res})      # noqa: E731
  for s, p in enumerate(prompts[:3]):
    state = proc.process(state, s, f"r{s}", p, 8, done)
  state = proc.flush(state, done)
  assert proc.passes == 2 and set(got) == {"r0", "r1", "r2"}
  first, _ = PrefillProcessor(eng).process(eng.init_decode_state(3), 0, prompts[1])
  assert int(first.data[0, 0]) == got["r1"]
  with pytest.raises(ValueError):
    proc.process(state, 0, "big", list(range(9)), 8)


def test_mmlu_prompt_parsing_grouping_and_both_scoring_modes(tmp_path):
  import json
  from maxtext_b200.benchmarks.mmlu import mmlu_eval as M
  from maxtext_b200.benchmarks.mmlu.subjects import AREA_OF, FIELD_OF
  from maxtext_b200.input_pipeline.tokenizer import ByteTokenizer
  assert len(FIELD_OF) == 57 and FIELD_OF["college_computer_science"] == "computer science" and AREA_OF["law"] == "humanities"
  p = M.construct_prompt("high_school_physics", "What falls?", ["Up", "Apples", "Nothing", "Sky"])
  assert "about high school physics." in p and "B. Apples" in p and p.endswith("Answer:")
  assert M.parse_answer("Answer: c because") == "C" and M.parse_answer("so The answer is (B).") == "B" and M.parse_answer("no idea") is None
  f = tmp_path / "mmlu.jsonl"
  rows = [{"subject": "anatomy", "question": f"q{i}", "choices": ["a", "b", "c", "d"], "answer": "ABCD"[i % 4] if i % 2 else i % 4} for i in range(6)]
  f.write_text("\n".join(json.dumps(r) for r in rows))
  samples = M.load_samples(str(f), limit=5)
  assert len(samples) == 5 and samples[1]["answer"] == 1 and samples[2]["answer"] == 2
  eng, cfg = _engine(extra=["vocab_size=300", "max_prefill_predict_length=40", "max_target_length=64"])
  tok = ByteTokenizer()
  for mode in ("loglik", "generate"):
    rep = M.evaluate(eng, tok, samples, mode=mode, max_new_tokens=3)
    assert rep["total"] == 5 and 0.0 <= rep["accuracy"] <= 1.0 and set(rep["subject"]) == {"anatomy"} and set(rep["area"]) == {"other (business, health, misc.)"}
  t = M.Tally()
  t.add("astronomy", True)
  t.add("astronomy", False)
  t.add("jurisprudence", True)
  r = t.report()
  assert r["accuracy"] == 2 / 3 and r["subject"]["astronomy"] == 0.5 and r["area"] == {"STEM": 0.5, "humanities": 1.0}
