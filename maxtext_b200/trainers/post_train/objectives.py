"""Post-training objectives expressed as per-token weights on the token losses.

The training engine differentiates sum_t w_t * xent_t. Several objectives are linear in the sequence
log-probabilities once their scalar coefficients are frozen, so their exact gradient is obtained by choosing w:

  SFT   w = 1 on completion tokens (prompt tokens 0 when sft_train_on_completion_only)
  DPO   loss = -log sigmoid(beta * ((pi_c - pi_r) - (ref_c - ref_r)));  d loss = -beta*sigmoid(-beta*delta) * d(pi_c - pi_r)
        with log pi(seq) = -sum_t xent_t:  w = +g on chosen tokens, -g on rejected tokens, g = beta * sigmoid(-beta*delta)
  GRPO  loss = -mean_t A * min(ratio, clip(ratio)) ; w = A * ratio on tokens whose ratio is inside the trust region
        (or whose clipping is inactive for the sign of A), 0 elsewhere; w multiplies xent = -log pi, hence the sign.
(src/maxtext/trainers/post_train/{sft,dpo,rl}; src/maxtext/experimental/rl/grpo_trainer.py)
"""
from __future__ import annotations

import torch


def sft_mask(prompt_len: torch.Tensor, total_len: torch.Tensor, S: int, completion_only: bool = True) -> torch.Tensor:
  """[B, S] target weights: target position t predicts token t+1."""
  t = torch.arange(S)[None]
  valid = t < (total_len[:, None] - 1)
  if completion_only:
    valid = valid & (t >= (prompt_len[:, None] - 1))
  return valid.float()


def sequence_logprob(token_losses: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
  return -(token_losses * mask).sum(-1)


def dpo_weights(pi_c, pi_r, ref_c, ref_r, mask_c, mask_r, beta: float = 0.1, label_smoothing: float = 0.0):
  """Returns (loss per pair, weights for chosen rows, weights for rejected rows, reward accuracy)."""
  delta = (pi_c - pi_r) - (ref_c - ref_r)
  loss = -(1 - label_smoothing) * torch.nn.functional.logsigmoid(beta * delta) - label_smoothing * torch.nn.functional.logsigmoid(-beta * delta)
  g = beta * ((1 - label_smoothing) * torch.sigmoid(-beta * delta) - label_smoothing * torch.sigmoid(beta * delta))
  return loss, g[:, None] * mask_c, -g[:, None] * mask_r, (delta > 0).float().mean()


def grpo_advantages(rewards: torch.Tensor, group_size: int, eps: float = 1e-6) -> torch.Tensor:
  """Group-relative advantages: (r - mean_group) / (std_group + eps); rewards [N] with N = groups * group_size."""
  r = rewards.view(-1, group_size)
  return ((r - r.mean(1, keepdim=True)) / (r.std(1, keepdim=True) + eps)).reshape(-1)


def grpo_weights(token_losses, old_token_losses, advantages, mask, clip: float = 0.2):
  """token losses are -log pi per token. Returns (surrogate loss, per-token weights for the engine)."""
  ratio = torch.exp(old_token_losses - token_losses)
  A = advantages[:, None]
  unclipped = ratio * A
  clipped = ratio.clamp(1 - clip, 1 + clip) * A
  surrogate = -(torch.minimum(unclipped, clipped) * mask).sum() / mask.sum().clamp_min(1)
  active = (unclipped <= clipped).float()               # gradient flows only where the unclipped term is the minimum
  return surrogate, A * ratio * active * mask


def gspo_weights(token_losses, old_token_losses, advantages, mask, clip: float = 0.2):
  """GSPO-token (`loss_algo: gspo-token`, src/maxtext/configs/post_train/rl.yml:52): the importance ratio is one number per
  sequence, s_i = exp(mean_t(log pi - log pi_old)), used (and clipped) for all of its tokens; the gradient still flows
  through each token's own probability, d s_it / d log pi_t = s_i. Returns (surrogate loss, per-token weights)."""
  n = mask.sum(1).clamp_min(1)
  s = torch.exp(((old_token_losses - token_losses) * mask).sum(1) / n)[:, None]          # [N, 1]
  A = advantages[:, None]
  unclipped = s * A
  clipped = s.clamp(1 - clip, 1 + clip) * A
  per_tok = torch.minimum(unclipped, clipped).expand_as(mask)
  surrogate = -(per_tok * mask).sum() / mask.sum().clamp_min(1)
  active = (unclipped <= clipped).float()
  return surrogate, (A * s * active).expand_as(mask) * mask


def distillation_loss(student_logits, teacher_logits, targets, mask, alpha: float = 0.5, temperature: float = 1.0):
  """alpha * CE(targets) + (1 - alpha) * T^2 * KL(teacher_T || student_T), mean over masked tokens
  (src/maxtext/trainers/post_train/distillation/distillation_utils.py)."""
  ce = torch.nn.functional.cross_entropy(student_logits.float(), targets, reduction="none")
  t = temperature
  p_t = torch.softmax(teacher_logits.float() / t, -1)
  kl = (p_t * (torch.log_softmax(teacher_logits.float() / t, -1) - torch.log_softmax(student_logits.float() / t, -1))).sum(-1)
  per_tok = alpha * ce + (1 - alpha) * t * t * kl
  return (per_tok * mask).sum() / mask.sum().clamp_min(1)
