"""Weight conversion against HuggingFace reference models built in-process (random weights, no download): logits of
the converted model must equal HF's, for both RoPE lane conventions, and the export must round-trip."""
import pytest
import torch

from helpers import BASE_YML
from maxtext_b200.checkpoint_conversion import hf as conv
from maxtext_b200.config import pyconfig
from maxtext_b200.models.transformer import Transformer

transformers = pytest.importorskip("transformers")


def _cfg(extra=()):
  return pyconfig.initialize(
      ["t", BASE_YML, "model_name=llama3-8b", "override_model_config=true", "base_emb_dim=64", "base_num_query_heads=4", "base_num_kv_heads=2",
       "head_dim=16", "base_mlp_dim=128", "base_num_decoder_layers=2", "vocab_size=128", "max_target_length=24", "dtype=float32",
       "hardware=cpu", "log_config=false", "rope_max_timescale=10000", *extra], num_devices=1)


def _hf_llama(cfg, rope_scaling=None):
  hc = transformers.LlamaConfig(hidden_size=cfg.emb_dim, intermediate_size=cfg.mlp_dim, num_hidden_layers=cfg.num_decoder_layers,
                                num_attention_heads=cfg.num_query_heads, num_key_value_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                                vocab_size=cfg.vocab_size, rms_norm_eps=cfg.normalization_layer_epsilon, rope_theta=float(cfg.rope_max_timescale),
                                max_position_embeddings=8192, tie_word_embeddings=False, attention_bias=False, rope_scaling=rope_scaling)
  torch.manual_seed(0)
  return transformers.LlamaForCausalLM(hc).float().eval()


@pytest.mark.parametrize("rope", ["default", "llama3.1"])
def test_converted_llama_matches_hf_logits(rope):
  cfg = _cfg([f"rope_type={rope}"])
  scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
             "original_max_position_embeddings": 8192} if rope == "llama3.1" else None
  hf = _hf_llama(cfg, scaling)
  model = Transformer(cfg, None, "cpu")
  missing = conv.to_maxtext(hf.state_dict(), model.store, cfg)
  assert not missing
  toks = torch.randint(0, cfg.vocab_size, (2, 24))
  with torch.no_grad():
    want = hf(toks).logits
  got = model.forward(toks)
  assert (got - want).abs().max() < 2e-4, (got - want).abs().max()
  back = conv.to_hf(model.store, cfg)
  for k, v in hf.state_dict().items():
    assert torch.allclose(back[k], v.float(), atol=1e-5), k


def test_mixtral_conversion_matches_hf_logits():
  cfg = pyconfig.initialize(
      ["t", BASE_YML, "model_name=mixtral-8x7b", "override_model_config=true", "base_emb_dim=64", "base_num_query_heads=4", "base_num_kv_heads=2",
       "head_dim=16", "base_mlp_dim=96", "base_moe_mlp_dim=96", "base_num_decoder_layers=2", "vocab_size=128", "max_target_length=16",
       "num_experts=4", "num_experts_per_tok=2", "dtype=float32", "hardware=cpu", "log_config=false", "rope_max_timescale=10000"], num_devices=1)
  hc = transformers.MixtralConfig(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                  head_dim=16, vocab_size=128, rms_norm_eps=cfg.normalization_layer_epsilon, rope_theta=10000.0,
                                  num_local_experts=4, num_experts_per_tok=2, max_position_embeddings=64, tie_word_embeddings=False,
                                  sliding_window=None)
  torch.manual_seed(0)
  hf = transformers.MixtralForCausalLM(hc).float().eval()
  model = Transformer(cfg, None, "cpu")
  sd = hf.state_dict()
  assert not conv.to_maxtext(sd, model.store, cfg)
  toks = torch.randint(0, 128, (2, 16))
  with torch.no_grad():
    want = hf(toks).logits
  got = model.forward(toks)
  assert (got - want).abs().max() < 5e-4


def test_checkpoint_cli_roundtrip(tmp_path):
  from safetensors.torch import load_file, save_file
  cfg = _cfg()
  hf = _hf_llama(cfg)
  src = tmp_path / "hf"
  src.mkdir()
  save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, str(src / "model.safetensors"))
  step_dir = conv.convert_hf_to_checkpoint(str(src), cfg, str(tmp_path / "ckpt"))
  out = conv.convert_checkpoint_to_hf(step_dir, cfg, str(tmp_path / "export"))
  back = load_file(str(tmp_path / "export" / "model.safetensors"))
  for k, v in hf.state_dict().items():
    assert torch.allclose(back[k], v.float(), atol=1e-5), k



def test_vllm_weight_stream_has_hf_names_and_values():
  """What an RL loop pushes into a vLLM rollout engine: one (HF name, tensor) pair per parameter, equal to the export."""
  from maxtext_b200.integration import vllm as mv
  from helpers import tiny_config, make_engine
  cfg = tiny_config("mixtral-8x7b", ["num_experts=4", "base_moe_mlp_dim=64"])
  eng = make_engine(cfg)
  want = conv.to_hf(eng.store, cfg)
  got = dict(mv.weights_iterator(eng.store, cfg))
  assert set(got) == set(want) and all(torch.equal(got[k], want[k]) for k in want)
  assert "model.layers.0.self_attn.q_proj.weight" in got and "model.layers.1.block_sparse_moe.experts.3.w2.weight" in got

  class FakeModel:
    def load_weights(self, it):
      self.names = [k for k, v in it if v.dtype == torch.bfloat16]
  fake = type("LLM", (), {})()
  fake.llm_engine = type("E", (), {})()
  fake.llm_engine.model_executor = type("X", (), {})()
  fake.llm_engine.model_executor.driver_worker = type("W", (), {})()
  fake.llm_engine.model_executor.driver_worker.model_runner = type("R", (), {"model": FakeModel()})()
  assert mv.sync_weights(fake, eng.store, cfg) == len(want)
