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

    def forward(self, input_ids, pos_xyz, example_ids=None, attention_mask=None, is_causal=True):
        eng = _resolve_engine(self.module, self._device)
        return forward_logits(eng, input_ids, pos_xyz, example_ids, attention_mask, is_causal)
