"""Full-sequence logits on the B200 engine with ``TinyTransformer.forward``'s signature
(``src/transformer.py:562-599``).  Inference only (no autograd)."""
from __future__ import annotations

import numpy as np
import torch

from .engine import Engine, plan_prefill
from .inference import DEFAULT_PREFILL_TOKENS, _resolve_engine


@torch.no_grad()
def forward_logits(model, input_ids: torch.Tensor, pos_xyz: torch.Tensor,
                   example_ids: torch.Tensor | None = None, attention_mask: torch.Tensor | None = None,
                   is_causal: bool = True, max_prefill_tokens: int = DEFAULT_PREFILL_TOKENS) -> torch.Tensor:
    """Logits ``[batch, seq, 14]`` (fp32) of every position.

    ``example_ids=None`` adds no example embedding, as in the reference forward.  With an
    ``attention_mask`` the keys of padded positions are excluded; padded query positions still
    get logits (computed from the valid keys they may see; zeros of attention when they see none).
    """
    engine = _resolve_engine(model, input_ids.device)
    B, S = input_ids.shape
    ids = input_ids.detach().cpu().numpy()
    pos = pos_xyz.detach().cpu().numpy()
    mask = (np.ones((B, S), dtype=bool) if attention_mask is None
            else attention_mask.detach().to(torch.bool).cpu().numpy())
    dev = engine.device
    per_call = max(1, max_prefill_tokens // max(S, 1))
    cap = min(B, per_call) * S
    session = engine.new_session(B, max(int(mask.sum(axis=1).max()), 1), 1, cap, stop_on_end=False)
    ex_dev = None
    if example_ids is not None and engine.use_example_embedding:
        ex_dev = example_ids.detach().to(device=dev, dtype=torch.int32).contiguous()
    out = torch.empty((B, S, 14), dtype=torch.float32, device=dev)
    for r0 in range(0, B, per_call):
        rows = np.arange(r0, min(B, r0 + per_call))
        plan = plan_prefill(ids, pos, mask, rows, is_causal=is_causal, all_positions=True, with_first=False)
        logits = torch.empty((plan.n_tokens, 14), dtype=torch.float32, device=dev)
        session.prefill(plan.to(dev), ex_dev, logits_all=logits)
        out[r0:r0 + len(rows)] = logits.view(len(rows), S, 14)
    session.poll()
    session.close()
    return out.to(input_ids.device) if input_ids.device.type == "cuda" else out.cpu()


class B200TinyTransformer(torch.nn.Module):
    """Wraps a reference ``TinyTransformer`` so that calling it runs the B200 engine.

    ``forward`` keeps the reference signature; parameters stay in the wrapped module (so
    ``state_dict``/checkpoints are unchanged) and are packed for the GPU on first use.
    """

    def __init__(self, module: torch.nn.Module, device="cuda:0"):
        super().__init__()
        self.module = module
        self.config = module.config
        self._device = torch.device(device)

    def __getattr__(self, name):
        # attributes of the wrapped module (num_parameters, token_embed, blocks, ...) read through
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("module"), name)

    def forward(self, input_ids, pos_xyz, example_ids=None, attention_mask=None, is_causal=True):
        eng = _resolve_engine(self.module, self._device)
        return forward_logits(eng, input_ids, pos_xyz, example_ids, attention_mask, is_causal)

    def reset_cache(self) -> None:
        """Nothing to reset: every call builds its own session (kept for callers of the reference API)."""

    @torch.no_grad()
    def generate(self, input_ids, pos_xyz, max_new_tokens, example_ids=None, temperature=1.0, top_k=None,
                 greedy=True):
        """The reference module's own ``generate`` (src/transformer.py:601-692), kept for its callers:
        every new token takes the last position with x advanced by one modulo ``max_x`` (no grid-state
        tracking, no END handling).  This is not the hot path (``generate_output`` is): each step
        recomputes the logits of the whole prefix on the engine, which is exact for a causal model."""
        ids, pos = input_ids, pos_xyz
        for _ in range(int(max_new_tokens)):
            logits = self.forward(ids, pos, example_ids)[:, -1, :]
            if greedy:
                nxt = logits.argmax(dim=-1, keepdim=True)
            else:
                probs = torch.softmax(logits / temperature, dim=-1)
                if top_k is not None:
                    v, _ = torch.topk(probs, min(top_k, probs.size(-1)))
                    probs = torch.where(probs < v[:, [-1]], torch.zeros_like(probs), probs)
                    probs = probs / probs.sum(dim=-1, keepdim=True)
                nxt = torch.multinomial(probs, num_samples=1)
            new_pos = pos[:, -1:, :].clone()
            new_pos[:, :, 0] = (new_pos[:, :, 0] + 1) % int(self.config.max_x)
            ids = torch.cat([ids, nxt.to(ids.dtype)], dim=1)
            pos = torch.cat([pos, new_pos], dim=1)
        return ids
