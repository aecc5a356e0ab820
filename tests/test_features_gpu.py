"""Newer model features on a GPU in bf16 against the fp32 CPU run of the same configuration: hyper-connections, the engram
memory, the sparse-attention indexer with hash-routed layers, block diffusion; the Qwen3-VL / Omni towers run and stay finite."""
import pytest
import torch

from test_train_gpu import _cfg

pytestmark = pytest.mark.gpu

MLA = ["model_name=deepseek2-16b", "override_model_config=true", "base_num_decoder_layers=3", "first_num_dense_layers=1", "num_experts=4",
       "num_experts_per_tok=2", "base_moe_mlp_dim=256", "kv_lora_rank=64", "qk_nope_head_dim=128", "qk_rope_head_dim=64", "v_head_dim=128",
       "shared_experts=1"]

CASES = {
    "hyper_connections_and_engram": MLA + ["mhc_expansion_rate=2", "engram_layers=[1]", "engram_vocab_bases=[50,70]", "engram_max_ngram_size=3",
                                           "engram_num_heads=2", "engram_head_dim=64", "engram_kernel_size=3", "tokenizer_type=byte"],
    "indexer_and_hash_routing": MLA + ["q_lora_rank=64", "use_indexer=true", "indexer_topk=32", "indexer_n_heads=4", "indexer_head_dim=64",
                                       "indexer_loss_scaling_factor=0.1", "first_num_hash_layers=2", "first_num_dense_layers=0",
                                       "routed_score_func=sigmoid", "routed_bias=true"],
    "block_diffusion": ["attention_type=block_diffusion", "training_objective=block_diffusion", "causal_block_size=32",
                        "block_diffusion_mask_id=3", "packing=false"],
}


def _losses(cfg, device, steps=3):
  from maxtext_b200.input_pipeline.synthetic import SyntheticDataIterator
  from maxtext_b200.train.engine import TrainEngine
  eng = TrainEngine(cfg, None, torch.device(device))
  it = SyntheticDataIterator(cfg, pin=False)
  if cfg.training_objective == "block_diffusion":
    from maxtext_b200.diffusion.block_diffusion.batches import BlockDiffusionIterator
    it = BlockDiffusionIterator(cfg, it)
  return [float(eng.train_step(next(it))["learning/loss"]) for _ in range(steps)]


@pytest.mark.parametrize("case", sorted(CASES))
def test_feature_trains_on_gpu_and_tracks_cpu(case):
  from maxtext_b200.ops import backend
  E = backend.ext(required=True)
  gpu = _losses(_cfg(CASES[case] + ["hardware=gpu"]), "cuda", 3)
  assert E.kernel_status(True) == 0
  cpu = _losses(_cfg(CASES[case] + ["hardware=cpu", "dtype=float32"]), "cpu", 3)
  # the two runs draw their initial weights from different generators (CPU / CUDA); with a top-k key selection on top, the
  # sparse-attention case wanders further than the others (measured 0.18 at the third step)
  tol = 0.3 if case == "indexer_and_hash_routing" else 0.15
  assert all(abs(a - b) < tol for a, b in zip(gpu, cpu)), (gpu, cpu)
  assert gpu[-1] < gpu[0]


def test_qwen3_omni_towers_run_on_gpu():
  """Image and audio soft tokens enter a bf16 decoder on the GPU: finite logits that depend on both inputs."""
  from maxtext_b200.models.audio import conv_output_length
  from maxtext_b200.models.transformer import Transformer
  cfg = _cfg(["model_name=qwen3-omni-30b-a3b", "override_model_config=true", "hardware=gpu", "num_experts=4", "num_experts_per_tok=2",
              "base_moe_mlp_dim=256", "use_multimodal=true", "use_audio=true", "d_model_for_audio=128", "encoder_attention_heads_for_audio=2",
              "encoder_ffn_dim_for_audio=256", "encoder_layers_for_audio=2", "num_mel_bins_for_audio=32", "downsample_hidden_size_for_audio=16",
              "output_dim_for_audio=512", "max_source_positions_for_audio=64", "hidden_size_for_vit=128", "intermediate_size_for_vit=256",
              "num_attention_heads_for_vit=2", "num_hidden_layers_for_vit=2", "deepstack_visual_indexes_for_vit=[0]", "out_hidden_size_for_vit=512",
              "num_position_embeddings_for_vit=36", "patch_size_for_vit=4", "temporal_patch_size_for_vit=2", "spatial_merge_size_for_vit=2", "image_size_for_vit=16",
              "tokenizer_type=byte"])
  model = Transformer(cfg, None, torch.device("cuda"))
  model.store.initialize(seed=0)
  B, S, frames = 2, 64, 150
  K = conv_output_length(frames)
  g = torch.Generator().manual_seed(0)
  tokens = torch.randint(1, 200, (B, S), generator=g).cuda()
  amask = torch.zeros(B, S, dtype=torch.bool)
  amask[:, 2:2 + K] = True
  imask = torch.zeros(B, S, dtype=torch.bool)
  imask[:, 30:34] = True                                        # one 16 x 16 image -> 2 x 2 soft tokens
  audio = torch.randn(B, 32, frames, generator=g).cuda()
  images = torch.randn(B, 1, 3, 16, 16, generator=g).cuda()
  with torch.no_grad():
    a = model.forward(tokens, images=images, image_mask=imask.cuda(), audio=audio, audio_mask=amask.cuda())
    b = model.forward(tokens, images=images, image_mask=imask.cuda(), audio=audio * 2.0, audio_mask=amask.cuda())
    c = model.forward(tokens, images=images * 2.0, image_mask=imask.cuda(), audio=audio, audio_mask=amask.cuda())
  assert a.shape == (B, S, cfg.vocab_size) and torch.isfinite(a).all()
  assert not torch.allclose(a, b) and not torch.allclose(a, c)
  assert torch.allclose(a[:, :2], b[:, :2], atol=1e-3)          # causal: nothing before the clip changes
