"""tcgen05 flash attention (forward, dK/dV, dQ) against the fp32 PyTorch definition with autograd."""
import pytest
import torch

from maxtext_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _E():
  from maxtext_b200.ops import backend
  return backend.ext(required=True)


def _reference(q, k, v, seg, window, scale):
  B, S = q.shape[:2]
  pos = torch.arange(S, device=q.device)[None].expand(B, S)
  qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
  mask = ref.attention_mask(pos, pos, seg, seg, True, window)
  out, lse = ref.attention(qf, kf, vf, mask, scale, return_lse=True)
  return qf, kf, vf, out, lse


def _case(B, S, Hq, Hkv, D, seg_mode=None, window=0, scale=1.0, packed=True, seed=0):
  E = _E()
  g = torch.Generator(device="cuda").manual_seed(seed)
  if packed:
    qkv = (0.5 * torch.randn(B, S, Hq + 2 * Hkv, D, device="cuda", generator=g)).bfloat16()
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
  else:
    q = (0.5 * torch.randn(B, S, Hq, D, device="cuda", generator=g)).bfloat16()
    k = (0.5 * torch.randn(B, S, Hkv, D, device="cuda", generator=g)).bfloat16()
    v = (0.5 * torch.randn(B, S, Hkv, D, device="cuda", generator=g)).bfloat16()
  seg = None
  if seg_mode == "packed":
    seg = torch.ones(B, S, dtype=torch.int32, device="cuda")
    seg[:, S // 3:] = 2
    seg[:, (2 * S) // 3 + 5:] = 3
    seg[1, -17:] = 0     # padding tail
  assert E.flash_bwd_supported(q, k, v)
  out = torch.empty(B, S, Hq, D, device="cuda", dtype=torch.bfloat16)
  lse = torch.empty(B, Hq, S, device="cuda")
  E.flash_fwd(q, k, v, out, lse, seg, seg, None, None, None, scale, 0.0, True, window, 0, 0)
  torch.cuda.synchronize()
  assert E.kernel_status(True) == 0, "bounded wait timed out in the forward kernel"
  qf, kf, vf, ro, rl = _reference(q, k, v, seg, window, scale)
  valid = torch.ones(B, S, dtype=torch.bool, device="cuda") if seg is None else seg != 0
  err = (out.float() - ro)[valid].abs().max().item()
  assert err <= 2e-2, f"forward max err {err}"
  lerr = (lse.transpose(1, 2)[valid] - rl.transpose(1, 2)[valid]).abs().max().item()
  assert lerr <= 2e-2, f"lse max err {lerr}"
  dout = (torch.randn(B, S, Hq, D, device="cuda", generator=g)).bfloat16()
  if seg is not None:
    dout = dout * valid[:, :, None, None]
  ro.backward(dout.float())
  if packed:
    dqkv = torch.zeros_like(qkv)
    dq, dk, dv = dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hkv], dqkv[:, :, Hq + Hkv:]
  else:
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
  E.flash_bwd(dout, q, k, v, out, lse, dq, dk, dv, seg, seg, None, None, scale, 0.0, True, window, 0, 0)
  torch.cuda.synchronize()
  assert E.kernel_status(True) == 0, "bounded wait timed out in a backward kernel"
  for name, got, want in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
    gotf = got.float()
    if seg is not None:
      gotf, want = gotf[valid], want[valid]
    e = (gotf - want).abs().max().item()
    s = want.abs().max().item()
    assert e <= 3e-2 * max(1.0, s), f"{name}: max err {e} (scale {s})"


def test_flash_single_tile():
  _case(1, 128, 1, 1, 128)


def test_flash_causal_gqa_packed():
  _case(2, 384, 4, 2, 128)


def test_flash_long_rows_rescale():
  # 8 key tiles per late query row: the running maximum moves and O is rescaled in tensor memory
  _case(1, 1024, 2, 1, 128, scale=0.3)


def test_flash_head_dim_64():
  _case(2, 256, 4, 4, 64, packed=False)


def test_flash_segments_and_padding():
  _case(2, 384, 4, 2, 128, seg_mode="packed")


def test_flash_sliding_window():
  _case(1, 512, 2, 2, 128, window=200)


def test_packed_attention_autograd_path():
  """The op the decoder layer calls: rope + attention over the packed projection, forward and backward."""
  from maxtext_b200.ops import functional as F
  B, S, Hq, Hkv, D = 2, 256, 4, 2, 128
  qkv = (0.5 * torch.randn(B, S, Hq + 2 * Hkv, D, device="cuda")).bfloat16().requires_grad_(True)
  pos = torch.arange(S, device="cuda", dtype=torch.int32)[None].expand(B, S).contiguous()
  inv = ref.rope_inv_timescale(D, 1, 10000).cuda()
  out = F.packed_attention(qkv.clone(), pos, None, inv, Hq, Hkv)
  dout = torch.randn_like(out)
  out.backward(dout)
  # reference
  x = qkv.detach().float().requires_grad_(True)
  qr = ref.apply_rope(x[:, :, :Hq], pos, inv, False)
  kr = ref.apply_rope(x[:, :, Hq:Hq + Hkv], pos, inv, False)
  m = ref.attention_mask(pos, pos)
  ro = ref.attention(qr, kr, x[:, :, Hq + Hkv:], m)
  ro.backward(dout.float())
  assert (out.float() - ro).abs().max() <= 3e-2
  assert (qkv.grad.float() - x.grad).abs().max() <= 4e-2 * max(1.0, x.grad.abs().max().item())


@pytest.mark.parametrize("B,Hq,Hkv,D,window", [(3, 8, 2, 128, 0), (2, 16, 16, 64, 0), (4, 32, 8, 128, 96), (1, 4, 1, 128, 0)])
def test_decode_attention_matches_reference(B, Hq, Hkv, D, window):
  """Split-KV decode kernel on a slot-indexed cache vs the fp32 reference on the gathered rows, ragged lengths."""
  from maxtext_b200.ops import backend, reference as ref
  E = backend.ext(required=True)
  torch.manual_seed(0)
  slots, max_len = 6, 700
  kc = (torch.randn(slots, max_len, Hkv, D, device="cuda") * 0.5).bfloat16()
  vc = (torch.randn(slots, max_len, Hkv, D, device="cuda") * 0.5).bfloat16()
  q = (torch.randn(B, Hq, D, device="cuda") * 0.3).bfloat16()
  slot_ids = torch.randperm(slots, device="cuda")[:B].to(torch.int32)
  lengths = torch.tensor([1, 64, 333, 700][:B] if B <= 4 else None, device="cuda", dtype=torch.int32)
  out = torch.empty(B, Hq, D, device="cuda", dtype=torch.bfloat16)
  for splits in (1, 5):
    E.decode_attention(q, kc, vc, slot_ids, lengths, out, 1.0, 0.0, window, splits)
    for b in range(B):
      n = int(lengths[b])
      K, V = kc[slot_ids[b].long(), :n][None], vc[slot_ids[b].long(), :n][None]
      qpos = torch.tensor([[n - 1]], device="cuda")
      kpos = torch.arange(n, device="cuda")[None]
      m = ref.attention_mask(qpos, kpos, None, None, True, window)
      want = ref.attention(q[b][None, None], K, V, m, 1.0, 0.0)[0, 0]
      assert (out[b].float() - want.float()).abs().max() < 2e-2, (b, splits)


def _fwd_general(B, Sq, Skv, Hq, Hkv, Dqk, Dv, *, causal=True, window=0, chunk=0, softcap=0.0, sinks=False, seg=False, arrays=False,
                 scale=0.25, seed=0, grads=True):
  """Forward kernel against the fp32 definition for the general mask / shape forms (the public op of ops.functional)."""
  from maxtext_b200.ops import functional as F
  E = _E()
  g = torch.Generator(device="cuda").manual_seed(seed)
  q = (torch.randn(B, Sq, Hq, Dqk, device="cuda", generator=g)).bfloat16()
  k = (torch.randn(B, Skv, Hkv, Dqk, device="cuda", generator=g)).bfloat16()
  v = (torch.randn(B, Skv, Hkv, Dv, device="cuda", generator=g)).bfloat16()
  off = Skv - Sq
  pos_q = (torch.arange(Sq, device="cuda") + off)[None].expand(B, Sq).contiguous()
  pos_k = torch.arange(Skv, device="cuda")[None].expand(B, Skv).contiguous()
  seg_q = seg_k = None
  if seg:
    seg_k = torch.ones(B, Skv, dtype=torch.int32, device="cuda")
    seg_k[:, Skv // 3:] = 2
    seg_k[:, (2 * Skv) // 3 + 7:] = 3
    seg_k[-1, -9:] = 0
    seg_q = seg_k[:, off:].contiguous()
  sk = (torch.randn(Hq, device="cuda", generator=g) * 2.0) if sinks else None
  kw = {}
  if arrays:
    # keys are a shuffled-block view of a longer sequence: positions come from arrays (as under context parallelism)
    perm = torch.cat([torch.arange(Skv // 2, Skv), torch.arange(0, Skv // 2)]).cuda()
    k, v, pos_k = k[:, perm].contiguous(), v[:, perm].contiguous(), pos_k[:, perm].contiguous()
    if seg:
      seg_k = seg_k[:, perm].contiguous()
    kw = dict(kv_positions=pos_k, kv_segment_ids=seg_k)
  out, lse = F.attention_fwd(q, k, v, pos_q, seg_q, scale, softcap, window, causal, chunk=chunk, sinks=sk, **kw)
  torch.cuda.synchronize()
  assert E.kernel_status(True) == 0
  assert E.flash_fwd_supported(q, k, v)
  mask = ref.attention_mask(pos_q, pos_k, seg_q, seg_k, causal, window, chunk)
  ro, rl = ref.attention(q.float(), k.float(), v.float(), mask, scale, softcap, sinks=sk, return_lse=True)
  rows = mask.any(-1)[:, 0]                                    # rows with at least one visible key
  if sinks:
    rows = torch.ones_like(rows)
  err = (out.float() - ro)[rows].abs().max().item()
  assert err <= 2e-2, f"forward max err {err}"
  lerr = (lse.transpose(1, 2)[rows] - rl.transpose(1, 2)[rows]).abs().max().item()
  assert lerr <= 2e-2, f"lse max err {lerr}"
  if not sinks and (~rows).any():
    assert out.float()[~rows].abs().max().item() == 0.0        # fully masked rows give zeros, not NaN
  if not grads:
    return
  # backward through the public op (kernels where they cover the shape) against autograd of the fp32 definition
  dout = torch.randn(B, Sq, Hq, Dv, device="cuda", generator=g).bfloat16() * rows[:, :, None, None]
  ql, kl, vl = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
  skl = sk.detach().clone().requires_grad_(True) if sinks else None
  before = F.attention_fallbacks()
  o2 = F.attention(ql, kl, vl, pos_q, seg_q, scale, softcap, window, causal, chunk=chunk, sinks=skl, **kw)
  o2.backward(dout)
  torch.cuda.synchronize()
  assert E.kernel_status(True) == 0
  assert F.attention_fallbacks() == before, "the backward left the kernels"
  qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
  skf = sk.detach().clone().requires_grad_(True) if sinks else None
  ref.attention(qf, kf, vf, mask, scale, softcap, sinks=skf).backward(dout.float())
  pairs = [("dq", ql.grad, qf.grad), ("dk", kl.grad, kf.grad), ("dv", vl.grad, vf.grad)] + ([("dsinks", skl.grad, skf.grad)] if sinks else [])
  for name, got, want in pairs:
    e = (got.float() - want).abs().max().item()
    sc = want.abs().max().item()
    assert e <= 3e-2 * max(1.0, sc), f"{name}: max err {e} (scale {sc})"


def test_fwd_ragged_lengths_not_multiples_of_the_tile():
  _fwd_general(2, 333, 333, 4, 2, 128, 128)
  _fwd_general(1, 130, 130, 2, 2, 64, 64)
  _fwd_general(1, 100, 100, 2, 1, 128, 128, causal=False)


def test_fwd_more_keys_than_queries_bottom_right_causal():
  _fwd_general(2, 200, 712, 4, 2, 128, 128)
  _fwd_general(1, 256, 1024, 2, 2, 128, 128, window=300)


def test_fwd_mla_shape_192_128():
  _fwd_general(2, 384, 384, 4, 4, 192, 128, scale=0.07)
  _fwd_general(1, 257, 257, 2, 2, 192, 128, scale=0.07, seg=True)
  _fwd_general(1, 200, 600, 4, 2, 192, 128, scale=0.07, window=250)
  _fwd_general(1, 512, 512, 2, 1, 192, 128, scale=0.07, arrays=True)


def test_fwd_logit_softcap():
  _fwd_general(2, 384, 384, 4, 2, 128, 128, softcap=5.0, scale=0.5)


def test_fwd_sinks():
  _fwd_general(2, 300, 300, 4, 2, 64, 64, sinks=True, window=128)


def test_fwd_chunked_attention():
  _fwd_general(2, 640, 640, 4, 2, 128, 128, chunk=256)
  _fwd_general(1, 500, 500, 2, 2, 128, 128, chunk=192)
  _fwd_general(1, 512, 512, 2, 2, 128, 128, chunk=128, seg=True)       # packed rows: positions come from arrays


def test_fwd_key_positions_from_arrays_with_tile_skipping():
  _fwd_general(2, 512, 512, 4, 2, 128, 128, arrays=True)
  _fwd_general(1, 640, 640, 2, 2, 128, 128, arrays=True, seg=True, window=200)
  _fwd_general(1, 384, 384, 2, 1, 128, 128, arrays=True, causal=False)


def test_fwd_bitwise_repeatable():
  E = _E()
  torch.manual_seed(3)
  q, k, v = ((0.5 * torch.randn(2, 1024, 4, 128, device="cuda")).bfloat16() for _ in range(3))
  outs = []
  for _ in range(2):
    out = torch.empty_like(q)
    lse = torch.empty(2, 4, 1024, device="cuda")
    E.flash_fwd(q, k, v, out, lse, None, None, None, None, None, 1.0, 0.0, True, 0, 0, 0)
    outs.append((out, lse))
  assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
  assert E.kernel_status(True) == 0
