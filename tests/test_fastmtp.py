"""FastMTP head: semantics restated from the reference's description of its forward pass
(cppmega/megatron/fastmtp_layer.py:32-47 step weights, :266-373 loop): roll-and-mask teacher forcing, one shared
block applied K times, per-step mean CE over valid targets, normalised decay weights, detached trunk and LM head."""
import dataclasses
import math

import torch
import torch.nn.functional as F

from cppmega_b200.config.model import MTPConfig, nam56r_tiny
from cppmega_b200.models.fastmtp import IGNORE, FastMTPHead, step_weights


def _cfg(depth=3, decay=0.6):
    base = nam56r_tiny(seq_length=24)
    return dataclasses.replace(base, mtp=MTPConfig(num_layers=0, fastmtp=True, fastmtp_depth=depth, fastmtp_decay=decay))


class _Emb(torch.nn.Module):
    def __init__(self, vocab, hidden):
        super().__init__()
        self.word_embeddings = torch.nn.Embedding(vocab, hidden)


def test_step_weights_are_a_normalised_decay():
    w = step_weights(4, 0.5)
    assert abs(float(w.sum()) - 1.0) < 1e-6
    assert torch.allclose(w[1:] / w[:-1], torch.full((3,), 0.5))


def test_forward_equals_a_plain_restatement_and_detaches_trunk_and_head():
    torch.manual_seed(0)
    cfg = _cfg()
    B, S, H, V = 2, 24, cfg.hidden_size, cfg.vocab_size
    head = FastMTPHead(cfg, dtype=torch.float32, seed=1)
    emb = _Emb(V, H)
    lm_w = torch.randn(V, H, requires_grad=True) * 0.05
    lm_w.retain_grad()
    trunk = torch.randn(B, S, H, requires_grad=True)
    labels = torch.randint(0, V, (B, S))
    mask = torch.ones(B, S)
    mask[0, 5:9] = 0
    got = head(trunk, None, labels, mask, emb, lm_w.detach())

    # plain restatement
    h = trunk.detach()
    ids, tgt = labels.clone(), labels.masked_fill(mask == 0, IGNORE)
    total = 0.0
    w = step_weights(cfg.mtp.fastmtp_depth, cfg.mtp.fastmtp_decay)
    for k in range(cfg.mtp.fastmtp_depth):
        ids = torch.cat([ids[:, 1:], ids.new_zeros(B, 1)], dim=1)
        tgt = torch.cat([tgt[:, 1:], tgt.new_full((B, 1), IGNORE)], dim=1)
        e = emb.word_embeddings(ids)
        x = torch.cat([F.rms_norm(h, (H,), eps=cfg.norm_eps), F.rms_norm(e, (H,), eps=cfg.norm_eps)], dim=-1)
        h = F.rms_norm(head.shared_block(head.proj(x)), (H,), eps=cfg.norm_eps)
        logits = h.reshape(B * S, H) @ lm_w.detach().t()
        total = total + w[k] * F.cross_entropy(logits, tgt.reshape(-1), ignore_index=IGNORE, reduction="mean")
    assert abs(float(got) - float(total)) < 1e-4 * max(1.0, abs(float(total)))
    assert math.isfinite(float(got)) and float(got) > 0

    got.backward()
    assert trunk.grad is None and lm_w.grad is None            # detached trunk and LM head
    assert head.proj.weight.grad is not None and head.proj.weight.grad.abs().sum() > 0
    assert emb.word_embeddings.weight.grad is not None          # teacher-forced embeddings train through the head


def test_model_adds_lambda_times_fastmtp_loss():
    from cppmega_b200.models import build_model
    from cppmega_b200.parallel.state import single_process_context
    torch.manual_seed(0)
    cfg = _cfg(depth=2)
    model = build_model(cfg, single_process_context())
    ids = torch.randint(0, cfg.vocab_size, (2, 24))
    out = model(ids, torch.roll(ids, -1, 1), None)
    cfg0 = dataclasses.replace(cfg, mtp=dataclasses.replace(cfg.mtp, fastmtp_lambda=0.0))
    model0 = build_model(cfg0, single_process_context())
    model0.load_state_dict(model.state_dict())
    out0 = model0(ids, torch.roll(ids, -1, 1), None)
    extra = float(out["loss"]) - float(out0["loss"])
    assert abs(float(out0["lm_loss"]) - float(out["lm_loss"])) < 1e-5
    assert extra > 0 and abs(extra / cfg.mtp.fastmtp_lambda - math.log(cfg.vocab_size)) < 2.0
