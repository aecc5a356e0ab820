"""Published checkpoints that ship quantised weights -> plain bf16 / fp32 safetensors that the converter reads
(src/maxtext/checkpoint_conversion/standalone_scripts/dequantize_mxfp4.py for GPT-OSS, deepseek_dequantize.py for DeepSeek-V3).

  MXFP4 (GPT-OSS experts): `<name>_blocks` uint8 [..., groups, 16] holds 32 four-bit E2M1 numbers per group (low nibble first),
    `<name>_scales` uint8 [..., groups] the group's power-of-two scale (E8M0, bias 127). Result `<name>` [..., groups * 32].
  FP8 block scaling (DeepSeek-V3): `<name>.weight` float8_e4m3fn [out, in] with `<name>.weight_scale_inv` fp32
    [ceil(out / 128), ceil(in / 128)]: every 128 x 128 tile is multiplied by its entry.

  python -m maxtext_b200.checkpoint_conversion.dequantize --input-path <dir> --output-path <dir> [--dtype bf16|fp16|fp32]
walks every *.safetensors file of a HuggingFace directory, rewrites the quantised tensors and the weight map in
`model.safetensors.index.json`, and copies everything else.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import shutil
import sys

import torch

# value of every E2M1 code: sign bit 3, exponent bits 2..1, mantissa bit 0 (0, 0.5, 1, 1.5, 2, 3, 4, 6 and their negatives)
E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])
BLOCK = 128


def dequantize_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
  lut = E2M1.to(blocks.device)
  b = blocks.to(torch.uint8)
  vals = torch.stack([lut[(b & 0xF).long()], lut[(b >> 4).long()]], -1)                 # [..., groups, 16, 2]: low nibble first
  scale = torch.exp2(scales.to(torch.float32) - 127.0)[..., None, None]
  return (vals * scale).reshape(*blocks.shape[:-2], -1).to(dtype)


def quantize_mxfp4(w: torch.Tensor):
  """The inverse, for tests and exports: [..., n] (n a multiple of 32) -> (blocks uint8 [..., n / 32, 16], scales uint8 [..., n / 32])."""
  g = w.float().reshape(*w.shape[:-1], -1, 32)
  amax = g.abs().amax(-1).clamp_min(2.0 ** -126)
  e = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)                              # largest magnitude maps inside +-6
  x = g / torch.exp2(e)[..., None]
  pos = E2M1[:8].to(w.device)
  idx = (x.abs()[..., None] - pos).abs().argmin(-1)
  code = (idx + 8 * (x < 0)).to(torch.uint8)
  blocks = (code[..., 0::2] | (code[..., 1::2] << 4)).to(torch.uint8)
  return blocks, (e + 127).to(torch.uint8)


def dequantize_fp8_blocks(weight: torch.Tensor, scale_inv: torch.Tensor, dtype=torch.bfloat16, block: int = BLOCK) -> torch.Tensor:
  out_f, in_f = weight.shape
  s = scale_inv.float().repeat_interleave(block, 0)[:out_f].repeat_interleave(block, 1)[:, :in_f]
  return (weight.float() * s).to(dtype)


def dequantize_state(state: dict, dtype=torch.bfloat16) -> tuple[dict, list]:
  """Returns (new state dict, names of the tensors that were rewritten)."""
  out, done = {}, []
  for k, v in state.items():
    if k.endswith("_scales") and k[:-7] + "_blocks" in state or k.endswith(".weight_scale_inv"):
      continue
    if k.endswith("_blocks") and k[:-7] + "_scales" in state:
      out[k[:-7]] = dequantize_mxfp4(v, state[k[:-7] + "_scales"], dtype)
      done.append(k[:-7])
    elif k.endswith(".weight") and k + "_scale_inv" in state and v.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
      out[k] = dequantize_fp8_blocks(v, state[k + "_scale_inv"], dtype)
      done.append(k)
    else:
      out[k] = v
  return out, done


def convert_directory(src: str, dst: str, dtype=torch.bfloat16) -> dict:
  from safetensors.torch import load_file, save_file
  os.makedirs(dst, exist_ok=True)
  files = sorted(glob.glob(os.path.join(src, "*.safetensors")))
  index_path = os.path.join(src, "model.safetensors.index.json")
  index = json.load(open(index_path)) if os.path.isfile(index_path) else None
  # a scale may sit in another shard than its weight: collect the companions first
  companions = {}
  for f in files:
    st = load_file(f)
    companions.update({k: v for k, v in st.items() if k.endswith(("_scales", ".weight_scale_inv"))})
  rewritten, weight_map = [], {}
  for f in files:
    st = load_file(f)
    merged = {**{k: companions[k] for k in companions if (k[:-7] + "_blocks" in st) or (k[:-10] in st)}, **st}
    new, done = dequantize_state(merged, dtype)
    new = {k: v.contiguous() for k, v in new.items() if k in done or k in st}
    save_file(new, os.path.join(dst, os.path.basename(f)), metadata={"format": "pt"})
    rewritten += done
    weight_map.update({k: os.path.basename(f) for k in new})
  if index is not None:
    index["weight_map"] = weight_map
    with open(os.path.join(dst, "model.safetensors.index.json"), "w") as fh:
      json.dump(index, fh, indent=1)
  for f in glob.glob(os.path.join(src, "*")):
    if os.path.isfile(f) and not f.endswith(".safetensors") and os.path.basename(f) != "model.safetensors.index.json":
      shutil.copy(f, os.path.join(dst, os.path.basename(f)))
  return {"files": len(files), "rewritten": len(rewritten)}


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--input-path", required=True)
  ap.add_argument("--output-path", required=True)
  ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
  a = ap.parse_args(argv)
  dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[a.dtype]
  print(json.dumps(convert_directory(a.input_path, a.output_path, dt)))
  return 0


if __name__ == "__main__":
  sys.exit(main())
