"""Worker for multi-GPU tests (one process per GPU, NCCL + symmetric memory). Writes 'ok' or a traceback to its result file."""
import os
import sys
import traceback

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def kernels(rank, world, dev):
  from maxtext_b200.ops import backend
  from maxtext_b200.parallel.symm import SymmGroup
  E = backend.ext(required=True)
  sg = SymmGroup(None, dev)
  # ---- fused reduce-scatter + sum of squares against a plain sum of the gathered buffers
  chunk = 3 * 1024 * 256
  full = sg.alloc(chunk * world, torch.float32)
  g = torch.Generator(device=dev).manual_seed(100 + rank)
  full.tensor.copy_(torch.randn(chunk * world, device=dev, generator=g))
  sg.barrier(1)
  dst = torch.zeros(chunk, device=dev)
  sq = torch.zeros(1, device=dev)
  E.rs_sumsq(full.table, rank * chunk, chunk, dst, False, 0.5, world, sq, 64)
  sg.barrier(2)
  gathered = [torch.empty(chunk * world, device=dev) for _ in range(world)]
  dist.all_gather(gathered, full.tensor)
  want = 0.5 * sum(t[rank * chunk:(rank + 1) * chunk] for t in gathered)
  assert torch.allclose(dst, want, atol=1e-5), (dst - want).abs().max()
  assert abs(sq.item() - want.double().pow(2).sum().item()) <= 1e-4 * want.numel()
  E.rs_sumsq(full.table, rank * chunk, chunk, dst, True, 0.5, world, None, 64)
  assert torch.allclose(dst, 2 * want, atol=1e-5)
  # ---- all-gather GEMM against all_gather + matmul
  N, K, M = 1024, 512, 640
  extra = 256 * 300                       # W does not start at the beginning of the unit
  unit = extra + N * K + 256 * 77
  c = -(-unit // (256 * world)) * 256
  shard = sg.alloc(c, torch.bfloat16)
  gw = torch.Generator(device=dev).manual_seed(7)
  whole = (0.1 * torch.randn(c * world, device=dev, generator=gw)).bfloat16()       # same on every rank
  shard.tensor.copy_(whole[rank * c:(rank + 1) * c])
  sg.barrier(3)
  fullbuf = torch.full((c * world,), float("nan"), device=dev, dtype=torch.bfloat16)
  flags = torch.zeros(world * 64, device=dev, dtype=torch.int32)
  a = (torch.randn(M, K, device=dev, generator=g)).bfloat16()
  out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
  E.gemm_ag(a, out, shard.table, fullbuf, N, K, c, 64 * 1024, extra, world, flags, 4)
  torch.cuda.synchronize()
  assert E.kernel_status(True) == 0
  assert torch.equal(fullbuf, whole), "gathered unit differs"
  ref = a.float() @ whole[extra:extra + N * K].view(N, K).float().t()
  assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max()
  # ---- stand-alone gather
  fullbuf.fill_(0)
  E.gather_segments(shard.table, fullbuf, c * 2, 128 * 1024, world, 8)
  torch.cuda.synchronize()
  assert torch.equal(fullbuf, whole)
  sg.barrier(4)
  sg.check()


def _canaries(fused):
  """Guard pages around every symmetric buffer must be intact after the steps (the test driver switches them on)."""
  from maxtext_b200.parallel import symm
  torch.cuda.synchronize()
  n = symm.verify_all_canaries()
  if fused and os.environ.get("MAXTEXT_B200_CANARIES") == "1":
    assert n > 0, "the fused path allocated no symmetric buffers"


def train_moe_ep(rank, world, dev, fused, extra=()):
  """Mixtral-style model with its experts spread over the `expert` axis: peer-memory dispatch vs the NCCL all-to-all path."""
  from maxtext_b200.config import pyconfig
  from maxtext_b200.parallel import mesh as mesh_lib
  from maxtext_b200.train import train as T
  from maxtext_b200.train.engine import TrainEngine
  cfg = pyconfig.initialize(
      ["w", "maxtext_b200/configs/base.yml", "model_name=mixtral-8x7b", "override_model_config=true", "base_emb_dim=512",
       "base_num_query_heads=4", "base_num_kv_heads=2", "head_dim=128", "base_mlp_dim=1024", "base_moe_mlp_dim=1024", "num_experts=8",
       "num_experts_per_tok=2", "base_num_decoder_layers=2", "vocab_size=4096", "max_target_length=256", "per_device_batch_size=2",
       "dataset_type=synthetic", "enable_checkpointing=false", "hardware=gpu", "weight_init=normal", "log_config=false", "steps=3",
       "learning_rate=1e-3", "warmup_steps_fraction=0.0", "ici_fsdp_parallelism=1", f"ici_expert_parallelism={world}",
       f"use_fused_comm_kernels={'true' if fused else 'false'}", *extra], num_devices=world)
  mesh = mesh_lib.mesh_from_config(cfg, rank=rank, world=world)
  eng = TrainEngine(cfg, mesh, dev)
  it = T.create_data_iterator(cfg, mesh)
  out = []
  for _ in range(3):
    m = eng.train_step(next(it))
    out.append((float(m["learning/loss"]), float(m["learning/raw_grad_norm"])))
  _canaries(fused)
  return out


def train_moe_ep_split(rank, world, dev, fused):
  """The same model with every layer run as two micro-batches on two streams (`use_batch_split_schedule`); the expert exchange
  of the split run goes through NCCL on both settings of `fused`. The balance loss is off so that the two runs agree exactly
  up to bf16 rounding (it is not linear in the batch)."""
  extra = ["load_balance_loss_weight=0.0"]
  if not fused:
    return train_moe_ep(rank, world, dev, False, extra)
  return train_moe_ep(rank, world, dev, True, extra + ["use_batch_split_schedule=true"])


def train_tp(rank, world, dev, fused):
  """Tensor parallelism over all ranks: all-reduces inside GEMM epilogues (peer-memory reduce-add) vs NCCL all-reduce."""
  from maxtext_b200.config import pyconfig
  from maxtext_b200.parallel import mesh as mesh_lib
  from maxtext_b200.train import train as T
  from maxtext_b200.train.engine import TrainEngine
  cfg = pyconfig.initialize(
      ["w", "maxtext_b200/configs/base.yml", "base_emb_dim=512", "base_num_query_heads=4", "base_num_kv_heads=2", "head_dim=128",
       "base_mlp_dim=1024", "base_num_decoder_layers=3", "vocab_size=4096", "max_target_length=256", "per_device_batch_size=2",
       "dataset_type=synthetic", "enable_checkpointing=false", "hardware=gpu", "weight_init=normal", "log_config=false", "steps=3",
       "learning_rate=1e-3", "warmup_steps_fraction=0.0", "ici_fsdp_parallelism=1", f"ici_tensor_parallelism={world}",
       f"use_fused_comm_kernels={'true' if fused else 'false'}"], num_devices=world)
  mesh = mesh_lib.mesh_from_config(cfg, rank=rank, world=world)
  eng = TrainEngine(cfg, mesh, dev)
  it = T.create_data_iterator(cfg, mesh)
  out = []
  for _ in range(3):
    m = eng.train_step(next(it))
    out.append((float(m["learning/loss"]), float(m["learning/raw_grad_norm"])))
  if fused:
    from maxtext_b200.parallel import tp_fused
    assert tp_fused._RT and all(rt.use > 0 for rt in tp_fused._RT.values()), "fused TP path did not run"
  _canaries(fused)
  return out


def train_fsdp_tp(rank, world, dev, fused):
  """fsdp (world / 2) x tensor 2: every sharded unit lives on the fsdp ranks of one tensor coordinate, a sub-group of the world.
  The fused collectives (symmetric memory over that sub-group) against NCCL on the same sub-group."""
  from maxtext_b200.config import pyconfig
  from maxtext_b200.parallel import mesh as mesh_lib
  from maxtext_b200.train import train as T
  from maxtext_b200.train.engine import TrainEngine
  cfg = pyconfig.initialize(
      ["w", "maxtext_b200/configs/base.yml", "base_emb_dim=512", "base_num_query_heads=4", "base_num_kv_heads=2", "head_dim=128",
       "base_mlp_dim=1024", "base_num_decoder_layers=3", "vocab_size=4096", "max_target_length=256", "per_device_batch_size=2",
       "dataset_type=synthetic", "enable_checkpointing=false", "hardware=gpu", "weight_init=normal", "log_config=false", "steps=3",
       "learning_rate=1e-3", "warmup_steps_fraction=0.0", f"ici_fsdp_parallelism={world // 2}", "ici_tensor_parallelism=2",
       f"use_fused_comm_kernels={'true' if fused else 'false'}"], num_devices=world)
  mesh = mesh_lib.mesh_from_config(cfg, rank=rank, world=world)
  eng = TrainEngine(cfg, mesh, dev)
  assert bool(eng.store.fused) == bool(fused), "the fused FSDP path should be on exactly when asked for"
  if fused:
    assert eng.store.symm.world == world // 2
  it = T.create_data_iterator(cfg, mesh)
  out = []
  for _ in range(3):
    m = eng.train_step(next(it))
    out.append((float(m["learning/loss"]), float(m["learning/raw_grad_norm"])))
  _canaries(fused)
  return out


def train_cp(rank, world, dev, strategy):
  """Context parallelism over all ranks (None: one rank alone on the whole batch). Every strategy must land on the flash
  kernels: the ring and all-gather forms attend to foreign key blocks through the kernels' position arrays."""
  from maxtext_b200.config import pyconfig
  from maxtext_b200.ops import functional as F
  from maxtext_b200.parallel import mesh as mesh_lib
  from maxtext_b200.train import train as T
  from maxtext_b200.train.engine import TrainEngine
  n = 1 if strategy is None else world
  par = [] if strategy is None else [f"ici_context_parallelism={world}", "ici_fsdp_parallelism=1", f"context_parallel_strategy={strategy}"]
  cfg = pyconfig.initialize(
      ["w", "maxtext_b200/configs/base.yml", "base_emb_dim=512", "base_num_query_heads=4", "base_num_kv_heads=2", "head_dim=128",
       "base_mlp_dim=1024", "base_num_decoder_layers=2", "vocab_size=4096", "max_target_length=1024",
       f"per_device_batch_size={2 * world if strategy is None else 2}",
       "dataset_type=synthetic", "enable_checkpointing=false", "hardware=gpu", "weight_init=normal", "log_config=false", "steps=3",
       "learning_rate=1e-3", "warmup_steps_fraction=0.0", "use_fused_comm_kernels=false"] + par, num_devices=n)
  mesh = mesh_lib.mesh_from_config(cfg, rank=rank, world=world) if strategy is not None else None
  eng = TrainEngine(cfg, mesh, dev)
  it = T.create_data_iterator(cfg, mesh)
  before = F.attention_fallbacks()
  out = []
  for _ in range(3):
    m = eng.train_step(next(it))
    out.append((float(m["learning/loss"]), float(m["learning/raw_grad_norm"])))
  assert F.attention_fallbacks() == before, f"{strategy}: attention fell back to PyTorch ops {F.attention_fallbacks() - before} times"
  return out


def train(rank, world, dev, fused):
  from maxtext_b200.config import pyconfig
  from maxtext_b200.parallel import mesh as mesh_lib
  from maxtext_b200.train import train as T
  from maxtext_b200.train.engine import TrainEngine
  cfg = pyconfig.initialize(
      ["w", "maxtext_b200/configs/base.yml", "base_emb_dim=512", "base_num_query_heads=4", "base_num_kv_heads=2", "head_dim=128",
       "base_mlp_dim=1024", "base_num_decoder_layers=3", "vocab_size=4096", "max_target_length=256", "per_device_batch_size=2",
       "dataset_type=synthetic", "enable_checkpointing=false", "hardware=gpu", "weight_init=normal", "log_config=false", "steps=3",
       "learning_rate=1e-3", "warmup_steps_fraction=0.0", f"use_fused_comm_kernels={'true' if fused else 'false'}"], num_devices=world)
  mesh = mesh_lib.mesh_from_config(cfg, rank=rank, world=world)
  eng = TrainEngine(cfg, mesh, dev)
  it = T.create_data_iterator(cfg, mesh)
  out = []
  for _ in range(3):
    m = eng.train_step(next(it))
    out.append((float(m["learning/loss"]), float(m["learning/raw_grad_norm"])))
  _canaries(fused)
  return out


def main():
  mode, result = sys.argv[1], sys.argv[2]
  rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
  try:
    from maxtext_b200.parallel import mesh as mesh_lib
    mesh_lib.init_distributed(timeout_s=120)
    dev = torch.device("cuda", torch.cuda.current_device())
    if mode == "kernels":
      kernels(rank, world, dev)
      msg = "ok"
    elif mode == "cp":
      ref = train_cp(rank, world, dev, None)
      got = {s: train_cp(rank, world, dev, s) for s in ("ring", "all_gather", "ulysses")}
      for s, vals in got.items():
        for (la, na), (lb, nb) in zip(ref, vals):
          assert abs(la - lb) < 3e-2 and abs(na - nb) < 5e-2 * max(1.0, na), (s, ref, vals)
      from maxtext_b200.ops import backend
      assert backend.ext().kernel_status(True) == 0
      msg = "ok " + repr((ref, got))
    else:
      fn = {"moe_ep": train_moe_ep, "moe_ep_split": train_moe_ep_split, "tp": train_tp, "fsdp_tp": train_fsdp_tp}.get(mode, train)
      a = fn(rank, world, dev, fused=False)
      b = fn(rank, world, dev, fused=True)
      for (la, na), (lb, nb) in zip(a, b):
        assert abs(la - lb) < 2e-2 and abs(na - nb) < 5e-2 * max(1.0, na), (a, b)
      from maxtext_b200.ops import backend
      assert backend.ext().kernel_status(True) == 0
      msg = "ok " + repr((a, b))
  except Exception:  # pylint: disable=broad-except
    msg = traceback.format_exc()
  with open(f"{result}.{rank}", "w") as fh:
    fh.write(msg)
  try:
    dist.destroy_process_group()
  except Exception:  # pylint: disable=broad-except
    pass


if __name__ == "__main__":
  main()
