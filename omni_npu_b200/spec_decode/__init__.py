"""Speculative decoding: proposers of draft tokens.  Verification lives in
``sample/rejection_sampler.py``; the scheduler carries drafts on the request."""
from .ngram_proposer import NgramProposer  # noqa: F401


def make_proposer(spec_cfg, runner=None):
    """Proposer for a ``SpeculativeConfig`` or None when speculation is off."""
    if spec_cfg is None or not spec_cfg.method or spec_cfg.num_speculative_tokens <= 0:
        return None
    if spec_cfg.method == "ngram":
        return NgramProposer(spec_cfg.num_speculative_tokens, spec_cfg.prompt_lookup_min,
                             spec_cfg.prompt_lookup_max)
    if spec_cfg.method in ("mtp", "deepseek_mtp"):
        from .mtp_proposer import MTPProposer
        return MTPProposer(runner, spec_cfg.num_speculative_tokens)
    raise ValueError(f"unknown speculative method {spec_cfg.method!r}")
