"""`python -m maxtext.inference.decode <config.yml> prompt="..."`: load -> prefill -> insert -> generate loop -> text
(src/maxtext/inference/decode.py:88-237)."""
from __future__ import annotations

import sys

import torch

from ..config import pyconfig
from ..input_pipeline.tokenizer import build_tokenizer
from ..utils import max_logging
from .maxengine import MaxEngine


def decode(config, prompt: str | None = None, engine: MaxEngine | None = None) -> str:
  eng = engine or MaxEngine(config)
  if engine is None:
    eng.load_params()
  tok = build_tokenizer(config)
  text_in = prompt if prompt is not None else config.prompt
  if bool(getattr(config, "use_chat_template", False)):
    # the prompt is one user turn; the template appends the header of the assistant's answer
    from ..input_pipeline import chat
    text_in = chat.render([{"role": "user", "content": text_in}], chat.load_template(config), add_generation_prompt=True)
  ids = tok.encode(text_in, add_bos=bool(config.add_bos))
  mm_kw = {}
  if bool(getattr(config, "use_multimodal", False)) and str(getattr(config, "image_path", "") or ""):
    # one <start_of_image> in the prompt per file of image_path; each grows to 260 positions (256 of them soft tokens)
    paths = [p for p in str(config.image_path).split(",") if p]
    if eng.model.vision.__class__.__name__ == "Qwen3VLVision":
      # <|vision_start|> <|image_pad|> x K <|vision_end|> per image, K from the resized image's patch grid
      from ..multimodal import processor_qwen3 as pq
      t_ids, mask, pix = pq.prepare(ids, paths, config)
    else:
      from ..multimodal import processor_gemma3 as pg
      if ids.count(pg.BEGIN_IMAGE_TOKEN) < len(paths):
        ids = ids + [pg.BEGIN_IMAGE_TOKEN] * (len(paths) - ids.count(pg.BEGIN_IMAGE_TOKEN))
      t_ids, mask, pix = pg.prepare(ids, paths, int(config.image_size_for_vit))
    ids = t_ids.tolist()
    mm_kw = dict(images=pix, image_mask=torch.nn.functional.pad(mask, (0, max(0, int(config.max_prefill_predict_length) - len(ids)))))
  if bool(getattr(config, "use_multimodal", False)) and bool(getattr(config, "use_audio", False)) and str(getattr(config, "audio_path", "") or ""):
    # one clip: <|audio_start|> <|audio_pad|> x K <|audio_end|>, K soft tokens from the clip's log-mel frames (16 kHz PCM .wav)
    from ..multimodal import processor_qwen3 as pq
    wave, sr = pq.read_wav(str(config.audio_path))
    if sr != 16000:
      raise ValueError(f"audio_path: the tower expects 16 kHz audio, the file has {sr} Hz")
    t_ids, amask, feats = pq.prepare_audio_prompt(ids, wave, config)
    ids = t_ids.tolist()
    pad_to = max(0, int(config.max_prefill_predict_length) - len(ids))
    mm_kw.update(audio=feats, audio_mask=torch.nn.functional.pad(amask, (0, pad_to)))
    if "image_mask" in mm_kw and mm_kw["image_mask"].numel() < len(ids) + pad_to:
      mm_kw["image_mask"] = torch.nn.functional.pad(mm_kw["image_mask"], (0, len(ids) + pad_to - mm_kw["image_mask"].numel()))
  ids = [i % config.vocab_size for i in ids][: int(config.max_prefill_predict_length)]
  n = len(ids)
  padded = torch.tensor(ids + [0] * (int(config.max_prefill_predict_length) - n), dtype=torch.long)
  prefix, first = eng.prefill(padded, n, **mm_kw)
  state = eng.insert(prefix, eng.init_decode_state(1), 0)
  out = [int(first.data[0, 0])]
  for _ in range(n, int(config.max_target_length) - 1):
    state, res = eng.generate(state)
    t = int(res.data[0, 0])
    out.append(t)
    if t == getattr(tok, "eos_id", -1) or not bool(state.active[0]):
      break
    stops = [x for x in (getattr(config, "stop_strings", None) or []) if x]
    if stops and any(x in tok.decode(out) for x in stops):
      break                                                   # `stop_strings`: generation ends once one of them appears
  text = tok.decode(out)
  for x in (getattr(config, "stop_strings", None) or []):
    if x and x in text:
      text = text[: text.index(x)]
  if config.autoregressive_decode_assert:
    assert text.startswith(config.autoregressive_decode_assert), f"generated {text!r}, expected prefix {config.autoregressive_decode_assert!r}"
  return text


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  config = pyconfig.initialize(argv)
  text = decode(config)
  max_logging.log(f"Input `{config.prompt}` -> `{text}`")
  return text


if __name__ == "__main__":
  main()
