"""Learn-to-init distillation of attention projections (src/maxtext/layers/learn_to_init_layer.py:37-439).

A student whose attention has fewer or narrower heads than its teacher starts from projections that are LINEAR MAPS OF THE
TEACHER'S: for q / k / v,  K_student[b, u, v] = sum_{x, y} C[b, x, y] A[x, u] B[y, v]  (C = frozen teacher kernel [emb, heads,
head_dim], A mixes heads, B mixes the head width), or with one general map W[x, y, u, v]; for the output projection the roles
of the axes are mirrored (C [heads, head_dim, emb]). Only A, B (or W) are trained in this phase, on the student's own loss;
afterwards the effective kernels are written into the student as ordinary weights ("collapse").

Here the phase is a small trainer around `TrainEngine`: every step it (1) forms the effective kernels and loads them into the
student's parameter store, (2) runs the student's forward / backward, which leaves d loss / d kernel in the gradient store,
(3) pushes those gradients through the einsum above to A, B / W and takes an Adam step on them. It runs on one process (the
maps are tiny; the student's own collectives are untouched).
"""
from __future__ import annotations

import math

import torch

PROJECTIONS = ("query", "key", "value", "out")


def effective_kernel(C: torch.Tensor, A=None, B=None, W=None, is_output: bool = False) -> torch.Tensor:
  """Reference-layout kernel of the student: [emb, u, v] for q / k / v, [u, v, emb] for the output projection."""
  if W is not None:
    return torch.einsum("xyb,xyuv->uvb", C, W) if is_output else torch.einsum("bxy,xyuv->buv", C, W)
  if is_output:
    return torch.einsum("yub,vy->uvb", torch.einsum("xyb,xu->yub", C, A), B)
  return torch.einsum("buy,yv->buv", torch.einsum("bxy,xu->buy", C, A), B)


class LearnToInit:
  """`teacher` maps a student parameter name ("layers_0/self_attention/query/kernel") to the teacher's kernel in REFERENCE
  layout ([emb, heads, head_dim]; [heads, head_dim, emb] for `out`). Layers not in `layer_indices` keep their own weights."""

  def __init__(self, engine, teacher: dict, general_map: bool = False, lr: float = 1e-2, layer_indices=None, seed: int = 0):
    self.eng, self.store = engine, engine.store
    assert getattr(engine, "inner_world", 1) == 1, "learn-to-init runs on one process"
    c = engine.config
    self.lr, self.t = float(lr), 0
    g = torch.Generator().manual_seed(seed)
    self.maps = {}
    for name, C in teacher.items():
      p = self.store.params[name]
      proj = name.split("/")[-2]
      assert proj in PROJECTIONS, name
      if layer_indices is not None and p.pdef.layer is not None and int(p.pdef.layer) not in set(layer_indices):
        continue
      is_out = proj == "out"
      ref_shape = tuple(p.pdef.ref_shape)                              # student kernel in reference layout
      C = C.detach().float().to(engine.device)
      if is_out:
        (u, v, emb), (x, y, emb_t) = ref_shape, tuple(C.shape)
      else:
        (emb, u, v), (emb_t, x, y) = ref_shape, tuple(C.shape)
      assert emb == emb_t, f"{name}: student and teacher widths differ ({emb} vs {emb_t})"

      def lecun(*shape, fan_in):
        return (torch.randn(*shape, generator=g) / math.sqrt(fan_in)).to(engine.device).requires_grad_(True)
      if general_map:
        train = {"W": lecun(x, y, u, v, fan_in=x * y)}
      else:
        train = {"A": lecun(x, u, fan_in=x), "B": lecun(v, y, fan_in=v) if is_out else lecun(y, v, fan_in=y)}
      self.maps[name] = dict(C=C, out=is_out, train=train, m={k: torch.zeros_like(t) for k, t in train.items()},
                             v={k: torch.zeros_like(t) for k, t in train.items()})
    # the 1/sqrt(head_dim) factor that some families fold into the query weights is part of the teacher's kernel already
    self._load_kernels()

  def kernel(self, name: str) -> torch.Tensor:
    m = self.maps[name]
    return effective_kernel(m["C"], m["train"].get("A"), m["train"].get("B"), m["train"].get("W"), m["out"])

  def _internal(self, name: str, k_ref: torch.Tensor) -> torch.Tensor:
    """reference [in..., out...] -> the store's [out, in] layout."""
    p = self.store.params[name]
    n_in = int(math.prod(p.pdef.ref_shape[:p.pdef.n_in_dims]))
    return k_ref.reshape(n_in, -1).t().contiguous()

  def _load_kernels(self):
    with torch.no_grad():
      for name in self.maps:
        self.store.load_full(name, self._internal(name, self.kernel(name)))
    self.store.sync_compute_from_master()

  def _kernel_grad(self, name: str) -> torch.Tensor:
    p = self.store.params[name]
    u = self.store.unit_of(p)
    off = u.offsets[u.params.index(p)]
    g = self.store.shard_view(u, self.store.grad_shard)[off: off + p.pdef.numel].view(p.pdef.shape).float()
    return g.t().reshape(p.pdef.ref_shape)                            # back to the reference layout

  def step(self, batch) -> dict:
    """One learn-to-init step: the student's loss is minimised over the maps only. Returns the engine's loss figures."""
    eng, store = self.eng, self.store
    eng.fwd_bwd(batch)
    store.finish_resident_grads()
    acc = eng._accum
    eng._accum = None
    inv_w = 1.0 / max(float(acc["weights"]), 1e-9)
    self.t += 1
    b1, b2, eps = 0.9, 0.999, 1e-8
    for name, m in self.maps.items():
      k = self.kernel(name)
      grads = torch.autograd.grad(k, list(m["train"].values()), self._kernel_grad(name) * inv_w)
      for (key, t), gr in zip(m["train"].items(), grads):
        m["m"][key].mul_(b1).add_(gr, alpha=1 - b1)
        m["v"][key].mul_(b2).addcmul_(gr, gr, value=1 - b2)
        mh, vh = m["m"][key] / (1 - b1 ** self.t), m["v"][key] / (1 - b2 ** self.t)
        with torch.no_grad():
          t.sub_(self.lr * mh / (vh.sqrt() + eps))
    store.grad_shard.zero_()
    self._load_kernels()
    return {"loss": float(acc["loss_sum"]) * inv_w, "weights": float(acc["weights"])}

  def collapse(self) -> dict:
    """Writes the final effective kernels into the student (they are ordinary weights from here on) and returns them."""
    self._load_kernels()
    return {name: self.kernel(name).detach() for name in self.maps}
