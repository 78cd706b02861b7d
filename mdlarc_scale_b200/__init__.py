"""B200-native greedy generation + AAIVR voting for the mdlARC_scale TinyTransformer.

Public API (same call signatures as the reference's ``src/inference.py`` / ``src/voting.py``):
``generate_output``, ``predict_with_augmentations``, ``predict_grid``, ``forward_logits``, ``aaivr_predict``,
``aggregate_votes``, ``compute_voting_stats``; and of ``src/eval.py``: ``evaluate_task``,
``evaluate_dataset``, ``generate_submission``.
"""
from .voting import aaivr_predict, aggregate_votes, compute_voting_stats, select_top_k  # noqa: F401

__all__ = ["generate_output", "predict_with_augmentations", "predict_grid", "forward_logits", "aaivr_predict",
           "aggregate_votes", "compute_voting_stats", "select_top_k", "Engine",
           "evaluate_task", "evaluate_dataset", "generate_submission"]


def __getattr__(name):  # torch-dependent parts are imported lazily
    if name in ("generate_output", "predict_with_augmentations", "predict_grid", "generate_tokens"):
        from . import inference
        return getattr(inference, name)
    if name in ("forward_logits", "B200TinyTransformer"):
        from . import transformer
        return getattr(transformer, name)
    if name in ("evaluate_task", "evaluate_dataset", "generate_submission"):
        from . import evaluation
        return getattr(evaluation, name)
    if name in ("Engine", "engine_for"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
