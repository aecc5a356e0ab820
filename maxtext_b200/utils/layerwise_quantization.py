"""Quantises a checkpoint one decoder layer at a time, for models whose full-precision weights do not fit on the host that
prepares them for serving.

  python -m maxtext_b200.utils.layerwise_quantization maxtext_b200/configs/base.yml model_name=deepseek2-16b \
      load_parameters_path=/ckpt/0/items quantization=int8 save_quantized_params_path=/ckpt/int8

The reference's tool loads and quantises DeepSeek checkpoints layer by layer with AQT (src/maxtext/utils/
layerwise_quantization.py:109-470). Here the parameter tree is walked from the configuration on the meta device (no
weights are allocated), every matrix of a layer is read on its own from the checkpoint arrays (`zarr3.read_array` with a
region, so a scanned checkpoint is sliced on disk), rounded to `bits`-bit integers with one scale per output channel, and
appended to `quantized_params.safetensors`; the peak host memory is one layer. The file is what
`checkpoint_is_quantized=true` loads (`MaxEngine.load_quantized_params`); tensors that stay in full precision
(embeddings, norms, routers) are still read from `load_parameters_path`."""
from __future__ import annotations

import os
import sys

import torch

from ..config import pyconfig
from ..utils import max_logging


def quantize_matrix(w: torch.Tensor, bits: int):
  qmax = float(2 ** (int(bits) - 1) - 1)
  scale = w.abs().amax(dim=-1, keepdim=True).clamp_(min=1e-12) / qmax
  return torch.clamp(torch.round(w / scale), -qmax, qmax).to(torch.int8), scale.squeeze(-1).float()


def layerwise_quantize(config, bits: int | None = None) -> dict:
  from safetensors.torch import save_file
  from ..checkpoint import manager as ckpt
  c = config
  bits = int(bits or (8 if c.quantization == "int8" else 4 if c.quantization == "int4" else 8))
  src = c.load_parameters_path
  assert src and c.save_quantized_params_path, "set load_parameters_path and save_quantized_params_path"
  items = os.path.join(src, "items") if os.path.isdir(os.path.join(src, "items")) else src
  # the parameter definitions only: the model is built on the meta device
  from ..models.transformer import Transformer
  import types
  model = Transformer(c, None, torch.device("meta"))
  view = types.SimpleNamespace(store=model.store, config=c, model=model)
  io = ckpt.TreeIO(view, None)
  store = model.store
  by_layer: dict = {}
  for name, p in store.params.items():
    d = p.pdef
    if d.layer is None or d.kind not in ("linear", "expert_linear") or len(d.shape) < 2:
      continue
    by_layer.setdefault((d.stack, d.layer), []).append((name, p))
  flat, n_bytes_in, n_bytes_out, peak = {}, 0, 0, 0
  for key in sorted(by_layer):
    layer_bytes = 0
    for name, p in by_layer[key]:
      w = io.read_param(items, ("params", "params"), p)
      if w is None:
        raise KeyError(f"{items} lacks {name}")
      w = w.float()
      layer_bytes += w.numel() * 4
      q, sc = quantize_matrix(w, bits)
      flat[name + "/q"], flat[name + "/scale"] = q.contiguous(), sc.contiguous()
      n_bytes_in += w.numel() * w.element_size()
      n_bytes_out += q.numel() + sc.numel() * 4
      del w
    peak = max(peak, layer_bytes)
    max_logging.log(f"layerwise quantization: {key[0]}_{key[1]} done ({len(by_layer[key])} matrices)")
  os.makedirs(c.save_quantized_params_path, exist_ok=True)
  out = os.path.join(c.save_quantized_params_path, "quantized_params.safetensors")
  save_file(flat, out)
  return {"file": out, "layers": len(by_layer), "matrices": len(flat) // 2, "bits": bits, "fp32_bytes": n_bytes_in, "quantized_bytes": n_bytes_out,
          "peak_layer_bytes": peak}


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  info = layerwise_quantize(pyconfig.initialize(argv))
  max_logging.log(f"wrote {info['file']}: {info['matrices']} matrices of {info['layers']} layers, "
                  f"{info['fp32_bytes'] / 2**20:.1f} MiB -> {info['quantized_bytes'] / 2**20:.1f} MiB")
  return info


if __name__ == "__main__":
  main()
