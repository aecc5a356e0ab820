"""Packing, shifting, file pipeline (jsonl) with rank sharding and iterator state, byte tokenizer."""
import json

import numpy as np

from helpers import tiny_config
from maxtext_b200.input_pipeline import packing
from maxtext_b200.input_pipeline.file_pipeline import FileDataIterator
from maxtext_b200.input_pipeline.tokenizer import ByteTokenizer


def test_first_fit_packing_and_shift():
  ex = [np.arange(1, 6), np.arange(10, 13), np.arange(20, 27), np.arange(30, 32)]
  rows = list(packing.pack_first_fit(ex, 9))
  assert len(rows) == 2
  assert rows[0]["tokens"].tolist() == [1, 2, 3, 4, 5, 10, 11, 12, 0]
  assert rows[0]["segmentation"].tolist() == [1, 1, 1, 1, 1, 2, 2, 2, 0]
  assert rows[0]["position"].tolist() == [0, 1, 2, 3, 4, 0, 1, 2, 0]
  assert rows[1]["tokens"].tolist()[:9] == [20, 21, 22, 23, 24, 25, 26, 30, 31]
  sh = packing.shift_for_lm(rows[0])
  assert sh["inputs"].tolist() == [1, 2, 3, 4, 5, 10, 11, 12] and sh["targets"].tolist() == [2, 3, 4, 5, 10, 11, 12, 0]
  assert sh["targets_segmentation"].tolist() == [1, 1, 1, 1, 0, 2, 2, 0]          # no loss across document boundaries
  assert len(list(packing.pack_first_fit(ex, 9, max_segments=1))) == 4


def test_concat_then_split():
  rows = list(packing.concat_then_split([np.arange(1, 8), np.arange(10, 18)], 5))
  assert [r["tokens"].tolist() for r in rows] == [[1, 2, 3, 4, 5], [6, 7, 10, 11, 12], [13, 14, 15, 16, 17]]
  assert rows[1]["segmentation"].tolist() == [1, 1, 2, 2, 2] and rows[1]["position"].tolist() == [5, 6, 0, 1, 2]


def test_file_pipeline_shards_and_resumes(tmp_path):
  f = tmp_path / "d.jsonl"
  with open(f, "w") as fh:
    for i in range(40):
      fh.write(json.dumps({"text": f"doc {i} " + "x" * (5 + i % 7)}) + "\n")
  args = ["dataset_type=hf", f"hf_train_files={f}", "per_device_batch_size=2", "max_target_length=16", "vocab_size=300", "packing=false",
          "num_epoch=1"]
  c = tiny_config("llama3-8b", args, num_devices=2)
  a, b = FileDataIterator(c, 0, 2), FileDataIterator(c, 1, 2)
  ba, bb = next(a), next(b)
  assert ba["inputs"].shape == (2, 16) and not np.array_equal(ba["inputs"].numpy(), bb["inputs"].numpy())
  tok = ByteTokenizer()
  assert tok.decode(ba["inputs"][0].tolist()).startswith("doc 0") and tok.decode(bb["inputs"][0].tolist()).startswith("doc 1")
  st = a.state()
  nxt = next(a)
  a2 = FileDataIterator(c, 0, 2)
  a2.load_state(st)
  assert np.array_equal(next(a2)["inputs"].numpy(), nxt["inputs"].numpy())
  packed = FileDataIterator(tiny_config("llama3-8b", args[:5] + ["packing=true", "num_epoch=1"], num_devices=1))
  row = next(packed)
  assert int(row["inputs_segmentation"].max()) >= 1 and (row["inputs_position"][row["inputs_segmentation"] == 0] == 0).all()


def test_rampup_batches_grow_without_skipping_samples():
  import torch
  from helpers import tiny_config
  from maxtext_b200.input_pipeline.interface import RampupIterator
  cfg = tiny_config(extra=["per_device_batch_size=8", "enable_rampup_batch_size=true", "per_device_batch_size_start=2",
                           "per_device_batch_size_increment=3", "global_rampup_samples=20"])
  assert cfg.rampup_end_step == 2

  class Counter:
    def __init__(self):
      self.n = 0

    def __next__(self):
      b = {"inputs": torch.arange(self.n, self.n + 8)[:, None].repeat(1, 4)}
      self.n += 8
      return b

  it = RampupIterator(cfg, Counter())
  sizes, seen = [], []
  for _ in range(12):
    b = next(it)
    sizes.append(b["inputs"].shape[0])
    seen += b["inputs"][:, 0].tolist()
  assert sizes[:5] == [2] * 5 and sizes[5:7] == [5, 5] and sizes[7:] == [8] * 5     # 10 samples per increment
  assert seen == list(range(len(seen)))                                              # contiguous stream: nothing lost or repeated


def test_rampup_trains_end_to_end():
  from helpers import tiny_config
  from maxtext_b200.train import train as train_lib
  cfg = tiny_config(extra=["per_device_batch_size=4", "enable_rampup_batch_size=true", "per_device_batch_size_start=2",
                           "per_device_batch_size_increment=2", "global_rampup_samples=4", "steps=4"])
  _, hist = train_lib.train_loop(cfg)
  toks = [int(h["learning/total_weights"]) for h in hist]
  assert toks[0] == 2 * cfg.max_target_length and toks[-1] == 4 * cfg.max_target_length


def test_use_sft_masks_prompt_tokens_through_packing(tmp_path):
  """`use_sft` with prompt / completion columns: one packed row holds several examples, and only completion tokens (and
  the end-of-sequence token) are targets when sft_train_on_completion_only is set."""
  import json
  from helpers import tiny_config
  from maxtext_b200.input_pipeline.interface import create_data_iterator
  p = tmp_path / "sft.jsonl"
  recs = [{"prompt": "abcd", "completion": "XY"}, {"prompt": "ef", "completion": "ZZZ"}, {"prompt": "ghi", "completion": "W"}] * 4
  p.write_text("\n".join(json.dumps(r) for r in recs))
  base = ["dataset_type=hf", f"hf_train_files={p}", "train_data_columns=['prompt','completion']", "tokenizer_type=byte", "vocab_size=260",
          "use_sft=true", "packing=true", "max_target_length=32", "per_device_batch_size=1", "add_bos=false", "add_eos=false"]
  b = next(create_data_iterator(tiny_config("llama3-8b", base + ["sft_train_on_completion_only=true"])))
  inp, tgt, tseg = b["inputs"][0].tolist(), b["targets"][0].tolist(), b["targets_segmentation"][0].tolist()
  text = bytes(t for t in inp if 0 < t < 256).decode()
  assert text.startswith("abcdXYefZZZghiW"[: len(text)]) or "abcdX" in text
  trained = bytes(t for t, s in zip(tgt, tseg) if s != 0 and 0 < t < 256).decode()
  assert set(trained) <= set("XYZW") and "Y" in trained and not set(trained) & set("abcdefghi")
  b2 = next(create_data_iterator(tiny_config("llama3-8b", base + ["sft_train_on_completion_only=false"])))
  trained2 = bytes(t for t, s in zip(b2["targets"][0].tolist(), b2["targets_segmentation"][0].tolist()) if s != 0 and 0 < t < 256).decode()
  assert set(trained2) & set("abcdefghi")


def test_data_shuffling_is_deterministic_resumable_and_complete(tmp_path):
  import json
  from helpers import tiny_config
  from maxtext_b200.input_pipeline.interface import create_data_iterator
  p = tmp_path / "d.jsonl"
  p.write_text("\n".join(json.dumps({"text": f"doc {i:03d}"}) for i in range(40)))
  base = ["dataset_type=hf", f"hf_train_files={p}", "tokenizer_type=byte", "vocab_size=260", "packing=false", "max_target_length=16",
          "per_device_batch_size=4", "enable_data_shuffling=true", "num_epoch=1"]

  def docs(it, n):
    out = []
    for _ in range(n):
      b = next(it)
      out += [bytes(t for t in row if 0 < t < 256).decode()[:7] for row in b["inputs"].tolist()]
    return out
  a = docs(create_data_iterator(tiny_config("llama3-8b", base)), 10)
  assert sorted(a) == [f"doc {i:03d}" for i in range(40)] and a != sorted(a)             # a permutation, not the file order
  assert a == docs(create_data_iterator(tiny_config("llama3-8b", base)), 10)              # same seed, same order
  assert a != docs(create_data_iterator(tiny_config("llama3-8b", base + ["data_shuffle_seed=5"])), 10)
  it = create_data_iterator(tiny_config("llama3-8b", base))
  first = docs(it, 3)
  st = it.state()
  it2 = create_data_iterator(tiny_config("llama3-8b", base))
  it2.load_state(st)
  assert first + docs(it2, 7) == a                                                         # resume continues the shuffled order
  # two data shards see disjoint halves of the same order
  r0 = docs(create_data_iterator(tiny_config("llama3-8b", base + ["per_device_batch_size=2"], num_devices=2), 0, 2), 10)
  r1 = docs(create_data_iterator(tiny_config("llama3-8b", base + ["per_device_batch_size=2"], num_devices=2), 1, 2), 10)
  assert sorted(r0 + r1) == sorted(a) and not set(r0) & set(r1)


def test_eval_uses_the_eval_files(tmp_path):
  import json
  from helpers import tiny_config, make_engine
  from maxtext_b200.train import train as T
  tr, ev = tmp_path / "train.jsonl", tmp_path / "eval.jsonl"
  tr.write_text("\n".join(json.dumps({"text": "aaaa bbbb cccc dddd"}) for _ in range(8)))
  ev.write_text("\n".join(json.dumps({"text": "zzzz yyyy xxxx wwww"}) for _ in range(8)))
  base = ["dataset_type=hf", f"hf_train_files={tr}", "tokenizer_type=byte", "vocab_size=260", "max_target_length=16", "per_device_batch_size=2",
          "eval_steps=1", "learning_rate=2e-2", "num_epoch=100"]
  cfg = tiny_config("llama3-8b", base + [f"hf_eval_files={ev}"])
  eng = make_engine(cfg)
  it = T.create_data_iterator(cfg, None)
  for _ in range(12):
    eng.train_step(next(it))                                  # memorise the training text
  held_out = T.run_eval(cfg, eng, None)
  on_train = T.run_eval(tiny_config("llama3-8b", base), eng, None)
  assert held_out > on_train + 0.5, (held_out, on_train)


def test_chat_template_rendering_and_sft_on_messages(tmp_path):
  import json
  from helpers import tiny_config
  from maxtext_b200.input_pipeline import chat
  from maxtext_b200.input_pipeline.interface import create_data_iterator
  msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}, {"role": "assistant", "content": "YO"}]
  assert chat.render(msgs[:2], chat.DEFAULT_TEMPLATE, True) == "system: be brief\nuser: hi\nassistant: "
  tpl = "{{ bos_token }}{% for m in messages %}<{{ m['role'] }}>{{ m['content'] }}</s>{% endfor %}{% if add_generation_prompt %}<assistant>{% endif %}"
  assert chat.split_for_sft(msgs, tpl) == ("<system>be brief</s><user>hi</s><assistant>", "YO")
  tf = tmp_path / "tpl.json"
  tf.write_text(json.dumps({"chat_template": tpl}))
  p = tmp_path / "chat.jsonl"
  p.write_text("\n".join(json.dumps({"messages": msgs}) for _ in range(4)))
  cfg = tiny_config("llama3-8b", ["dataset_type=hf", f"hf_train_files={p}", "train_data_columns=['messages']", "tokenizer_type=byte",
                                  "vocab_size=260", "use_sft=true", "sft_train_on_completion_only=true", "packing=false",
                                  "max_target_length=64", "per_device_batch_size=1", "add_bos=false", "add_eos=false",
                                  f"chat_template_path={tf}"])
  b = next(create_data_iterator(cfg))
  text = bytes(t for t in b["inputs"][0].tolist() if 0 < t < 256).decode()
  assert text.startswith("<system>be brief</s><user>hi</s><assistant>Y")
  trained = bytes(t for t, s in zip(b["targets"][0].tolist(), b["targets_segmentation"][0].tolist()) if s != 0 and 0 < t < 256).decode()
  assert trained == "YO"


def test_decode_wraps_prompt_with_chat_template(monkeypatch):
  from helpers import tiny_config
  from maxtext_b200.input_pipeline import tokenizer as tk
  from maxtext_b200.inference import decode as dec
  seen = []
  orig = tk.ByteTokenizer.encode

  def spy(self, text, *a, **k):
    seen.append(text)
    return orig(self, text, *a, **k)
  monkeypatch.setattr(tk.ByteTokenizer, "encode", spy)
  cfg = tiny_config("llama3-8b", ["tokenizer_type=byte", "vocab_size=260", "use_chat_template=true", "prompt=hi", "max_target_length=32",
                                  "max_prefill_predict_length=16", "per_device_batch_size=1", "chat_template=[{{ messages[0]['content'] }}]>"])
  dec.decode(cfg)
  assert seen and seen[0] == "[hi]>"


def _drain(it, n):
  return [next(it)["inputs"].numpy().copy() for _ in range(n)]


def test_resume_is_sample_exact_inside_a_packing_window_and_inside_a_token_file(tmp_path):
  """The reader runs up to a packing window ahead of what was delivered, and a .npy file is one example of many rows:
  the saved position must be that of the last delivered row in both cases."""
  f = tmp_path / "d.jsonl"
  with open(f, "w") as fh:
    for i in range(300):
      fh.write(json.dumps({"text": f"doc {i} " + "y" * (3 + (i * 7) % 23)}) + "\n")
  base = ["dataset_type=hf", f"hf_train_files={f}", "per_device_batch_size=2", "max_target_length=32", "vocab_size=300", "num_epoch=2"]
  for extra in (["packing=true"], ["packing=true", "grain_packing_type=concat_then_split"], ["packing=false"]):
    c = tiny_config("llama3-8b", base + extra, num_devices=2)
    for rank in (0, 1):
      ref = _drain(FileDataIterator(c, rank, 2), 9)
      it = FileDataIterator(c, rank, 2)
      _drain(it, 4)
      st = json.loads(json.dumps(it.state()))
      it2 = FileDataIterator(c, rank, 2)
      it2.load_state(st)
      got = _drain(it2, 5)
      assert all(np.array_equal(a, b) for a, b in zip(got, ref[4:])), (extra, rank)
  npy = tmp_path / "t.npy"
  np.save(npy, (np.arange(33 * 10 + 5) % 250).astype(np.int32))
  c = tiny_config("llama3-8b", ["dataset_type=olmo_grain", f"grain_train_files={npy}", "per_device_batch_size=2", "max_target_length=32",
                               "vocab_size=300", "packing=false", "num_epoch=1"], num_devices=1)
  ref = _drain(FileDataIterator(c), 4)
  it = FileDataIterator(c)
  _drain(it, 2)
  it2 = FileDataIterator(c)
  it2.load_state(it.state())
  assert all(np.array_equal(a, b) for a, b in zip(_drain(it2, 2), ref[2:]))


def test_rampup_resume_keeps_the_partially_used_buffer(tmp_path):
  from maxtext_b200.input_pipeline.interface import create_data_iterator
  f = tmp_path / "d.jsonl"
  with open(f, "w") as fh:
    for i in range(400):
      fh.write(json.dumps({"text": f"doc {i} " + "z" * (i % 11)}) + "\n")
  c = tiny_config("llama3-8b", ["dataset_type=hf", f"hf_train_files={f}", "per_device_batch_size=8", "max_target_length=16", "vocab_size=300",
                               "packing=false", "enable_rampup_batch_size=true", "per_device_batch_size_start=2",
                               "per_device_batch_size_increment=3", "global_rampup_samples=20"], num_devices=1)
  ref = _drain(create_data_iterator(c), 12)
  for stop in (1, 3, 7, 9):
    it = create_data_iterator(c)
    _drain(it, stop)
    st = json.loads(json.dumps(it.state()))
    it2 = create_data_iterator(c)
    it2.load_state(st)
    got = _drain(it2, 12 - stop)
    assert all(a.shape == b.shape and np.array_equal(a, b) for a, b in zip(got, ref[stop:])), stop


def test_tfrecord_example_and_arrow_readers(tmp_path):
  """TFRecord framing with checksums, tf.train.Example wire format and Arrow IPC files, without TensorFlow."""
  import numpy as np
  import pyarrow as pa
  import pytest
  from maxtext_b200.input_pipeline import record_formats as rf
  assert rf.crc32c(b"123456789") == 0xE3069283                        # the check value of CRC-32C
  rows = [{"text": "hello world", "ids": [1, 2, 3, -4, 2 ** 40], "score": [0.5, 1.5]}, {"text": "zweite Zeile äöü", "ids": [7], "score": [2.0]}]
  path = str(tmp_path / "c4-train.tfrecord-00000-of-00001")
  rf.write_tfrecord(path, [rf.build_example(r) for r in rows])
  back = list(rf.read_tfrecord_examples(path))
  assert [b["text"] for b in back] == [r["text"] for r in rows]
  assert back[0]["ids"].tolist() == rows[0]["ids"] and np.allclose(back[0]["score"], rows[0]["score"])
  assert len(list(rf.read_tfrecord(path, verify_payload=True))) == 2
  raw = bytearray(open(path, "rb").read())
  raw[3] ^= 0xFF                                                       # damage the first length field
  bad = str(tmp_path / "bad.tfrecord")
  open(bad, "wb").write(bytes(raw))
  with pytest.raises(IOError):
    list(rf.read_tfrecord(bad))
  raw = bytearray(open(path, "rb").read())
  raw[20] ^= 0x01                                                      # damage a payload byte
  open(bad, "wb").write(bytes(raw))
  with pytest.raises(IOError):
    list(rf.read_tfrecord(bad, verify_payload=True))
  table = pa.table({"text": ["a b c", "d e"], "n": [1, 2]})
  for kind in ("file", "stream"):
    ap = str(tmp_path / f"data_{kind}.arrow")
    with pa.OSFile(ap, "wb") as sink:
      w = (pa.ipc.new_file if kind == "file" else pa.ipc.new_stream)(sink, table.schema)
      w.write_table(table)
      w.close()
    assert list(rf.read_arrow(ap)) == [{"text": "a b c", "n": 1}, {"text": "d e", "n": 2}]


def test_file_pipeline_reads_tfrecord_shards_and_prefetch_keeps_resume_exact(tmp_path):
  import torch
  from helpers import tiny_config
  from maxtext_b200.input_pipeline import record_formats as rf
  from maxtext_b200.input_pipeline.interface import PrefetchIterator, create_data_iterator
  texts = [f"record number {i} " + "tok " * (3 + i % 7) for i in range(120)]
  for sh in range(2):
    rf.write_tfrecord(str(tmp_path / f"c4-train.tfrecord-0000{sh}-of-00002"), [rf.build_example({"text": t}) for t in texts[sh::2]])
  base = ["dataset_type=tfds", f"dataset_path={tmp_path}/c4-train.tfrecord-*", "tokenizer_type=byte", "vocab_size=260", "max_target_length=32",
          "per_device_batch_size=2", "packing=true", "num_epoch=1"]
  plain = create_data_iterator(tiny_config("llama3-8b", base + ["grain_worker_count=0"]))
  assert not isinstance(plain, PrefetchIterator)
  want = [b["inputs"].clone() for b in plain]
  assert len(want) > 6
  it = create_data_iterator(tiny_config("llama3-8b", base + ["grain_worker_count=2", "grain_per_worker_buffer_size=2"]))
  assert isinstance(it, PrefetchIterator)
  got = [next(it)["inputs"] for _ in range(3)]
  st = it.state()                                                      # the thread has read further ahead than three batches
  got += [b["inputs"] for b in it]
  assert len(got) == len(want) and all(torch.equal(a, b) for a, b in zip(got, want))
  it2 = create_data_iterator(tiny_config("llama3-8b", base + ["grain_worker_count=2", "grain_per_worker_buffer_size=2"]))
  it2.load_state(st)
  rest = [b["inputs"] for b in it2]
  assert len(rest) == len(want) - 3 and all(torch.equal(a, b) for a, b in zip(rest, want[3:]))
  it.close(), it2.close()


def test_streaming_huggingface_dataset_backend(tmp_path):
  """dataset_type=hf with hf_path: rows come from `datasets` in streaming mode; same batches as the plain file reader, and
  the buffered shuffle is reproducible across iterators (ranks, resumed runs)."""
  import json
  import pytest
  import torch
  pytest.importorskip("datasets")
  from helpers import tiny_config
  from maxtext_b200.input_pipeline.interface import create_data_iterator
  p = tmp_path / "corpus.jsonl"
  p.write_text("\n".join(json.dumps({"text": f"document {i} " + "word " * (2 + i % 5)}) for i in range(60)))
  base = ["dataset_type=hf", f"hf_train_files={p}", "tokenizer_type=byte", "vocab_size=260", "max_target_length=32", "per_device_batch_size=2",
          "packing=true", "num_epoch=1", "grain_worker_count=0"]
  plain = [b["inputs"].clone() for b in create_data_iterator(tiny_config("llama3-8b", base))]
  stream = [b["inputs"].clone() for b in create_data_iterator(tiny_config("llama3-8b", base + ["hf_path=json"]))]
  assert len(plain) == len(stream) > 3 and all(torch.equal(a, b) for a, b in zip(plain, stream))
  sh = base + ["hf_path=json", "enable_data_shuffling=true", "data_shuffle_seed=3"]
  a = [b["inputs"].clone() for b in create_data_iterator(tiny_config("llama3-8b", sh))]
  b2 = [b["inputs"].clone() for b in create_data_iterator(tiny_config("llama3-8b", sh))]
  assert all(torch.equal(x, y) for x, y in zip(a, b2)) and not all(torch.equal(x, y) for x, y in zip(a, plain))


def test_olmo_mix_index_sampler_filter_and_resume(tmp_path):
  """Flat token files -> windows, one seeded permutation per epoch split over the data ranks, repetitive windows masked, the
  reader position is the batch count."""
  import numpy as np
  import torch
  from helpers import tiny_config
  from maxtext_b200.input_pipeline import olmo_data as O
  from maxtext_b200.input_pipeline.interface import create_data_iterator
  S = 32
  rng = np.random.default_rng(0)
  a = rng.integers(5, 200, size=S * 5 + 7).astype(np.uint32)           # 5 windows, 7 tokens dropped
  b = rng.integers(5, 200, size=S * 4).astype(np.uint16)               # raw file, 4 windows
  b[S * 2: S * 3] = np.tile(np.array([9, 8], dtype=np.uint16), S // 2)  # window 2 of b: period 2 repeated 16 times
  b[S * 3: S * 4] = 7                                                   # window 3 of b: one token 32 times
  np.save(tmp_path / "a.npy", a)
  b.tofile(tmp_path / "b.bin")
  # files of different element types need separate calls for raw data: index them together through explicit entries
  ia = O.build_index([str(tmp_path / "a.npy")], S)
  ib = O.build_index([str(tmp_path / "b.bin")], S, "uint16")
  idx = O.MixIndex(S, ia.files + [O.FileEntry(**{**ib.files[0].__dict__, "instance_offset": ia.total_instances})])
  assert idx.total_instances == 9 and [f.n_instances for f in idx.files] == [5, 4] and idx.files[0].data_offset > 0
  f, start = idx.locate(6)
  assert f.path.endswith("b.bin") and start == S
  idx.save(str(tmp_path / "index.json"))
  again = O.load_index(str(tmp_path / "index.json"), str(tmp_path), "/elsewhere")
  assert again.files[0].path == "/elsewhere/a.npy" and again.fingerprint() == idx.fingerprint()
  # repetition filter
  assert O.longest_repetition(np.tile([1, 2, 3], 10)) == 10 and O.longest_repetition(np.arange(50)) == 1
  assert not O.is_clean_instance(np.full(40, 7)) and O.is_clean_instance(np.tile([9, 8], 16)) and not O.is_clean_instance(np.tile([9, 8], 32))
  # sampler: each epoch is a permutation split over the ranks, epochs differ
  s0, s1 = O.OlmoSampler(9, 3, 0, 2), O.OlmoSampler(9, 3, 1, 2)
  ep0 = [s0[i] for i in range(4)] + [s1[i] for i in range(4)]
  assert len(set(ep0)) == 8 and [s0[i] for i in range(4)] != [s0[4 + i] for i in range(4)]
  assert [O.OlmoSampler(9, 3, 0, 2)[i] for i in range(8)] == [s0[i] for i in range(8)]
  # iterator through the dispatcher
  cfg = tiny_config("llama3-8b", ["dataset_type=olmo_grain", f"olmo_index_path={tmp_path / 'index.json'}", f"max_target_length={S}",
                                  "per_device_batch_size=3", "enable_data_shuffling=false"])
  it = create_data_iterator(cfg)
  batches = [next(it) for _ in range(3)]
  flat = torch.cat([x["inputs"] for x in batches])
  assert flat.shape == (9, S) and torch.equal(flat[0], torch.from_numpy(a[:S].astype(np.int32)))
  assert torch.equal(batches[0]["targets"][0, :-1], batches[0]["inputs"][0, 1:]) and int(batches[0]["targets_segmentation"][0, -1]) == 0
  seg = torch.cat([x["targets_segmentation"] for x in batches])
  assert int(seg[8].sum()) == 0 and int(seg[7].sum()) == S - 1 and int(seg[0].sum()) == S - 1      # only the 32-fold repetition is masked
  st = it.state()
  nxt = next(it)
  it2 = create_data_iterator(cfg)
  it2.load_state(st)
  assert torch.equal(next(it2)["inputs"], nxt["inputs"])
  O.main(["--out", str(tmp_path / "cli.json"), "--sequence-length", str(S), str(tmp_path / "a.npy")])
  assert O.load_index(str(tmp_path / "cli.json")).total_instances == 5
