"""Which layer of a hybrid stack is Mamba ('M'), attention ('*') or MLP ('-').

Same results as the reference allocator (mamba2hybrid/mamba2hybrid_layer_allocation.py:38-170, itself
from Megatron-LM): attention layers are spread evenly with Mamba at both ends, then MLP layers are
spread evenly over the remaining Mamba slots, right-justified; an explicit pattern overrides both.
For (56, 0.08, 0.5) this yields
`M-M-M--M-M*-M-M-M-M--M*-M-M-M-M-M*--M-M-M-M-M*-M--M-M-M-` (24 M, 4 attention, 28 MLP).
"""
from __future__ import annotations

import logging
from typing import List, Optional

MAMBA, ATTENTION, MLP = "M", "*", "-"
VALID = (MAMBA, ATTENTION, MLP)
log = logging.getLogger(__name__)


def _spread(slots: List[str], eligible: str, period: float, mark: str) -> None:
    """Walk the slots holding `eligible` with an error accumulator that starts at `period`,
    drops by one per slot and, whenever it falls below one half, marks the slot and adds `period`."""
    acc = period
    for i, s in enumerate(slots):
        if s != eligible:
            continue
        if acc < 0.5:
            slots[i] = mark
            acc += period
        else:
            acc -= 1.0


def _auto(total: int, attention_ratio: float, mlp_ratio: float) -> List[str]:
    n_attn = round(total * attention_ratio)
    n_mlp = round(total * mlp_ratio)
    slots = [MAMBA] * total
    n_mamba = total - n_attn
    _spread(slots, MAMBA, n_mamba / (n_attn + 1), ATTENTION)
    if n_mlp > 0:
        _spread(slots, MAMBA, (n_mamba - n_mlp) / n_mlp, MLP)
    return slots


def _from_pattern(total: int, pattern: str) -> List[str]:
    slots = list(pattern)
    if len(slots) != total:
        raise ValueError(f"hybrid override pattern has {len(slots)} symbols, the model has {total} layers")
    bad = sorted(set(slots) - set(VALID))
    if bad:
        raise ValueError(f"hybrid override pattern contains {bad}; allowed symbols are {VALID}")
    return slots


def allocate_layers(total_layers_count: int, target_attention_ratio: float, target_mlp_ratio: float,
                    override_pattern: Optional[str] = None, verbose: bool = False) -> List[str]:
    if total_layers_count < 1:
        raise ValueError("need at least one layer")
    if not (0.0 <= target_attention_ratio <= 1.0 and 0.0 <= target_mlp_ratio <= 1.0):
        raise ValueError("ratios must lie in [0, 1]")
    if target_attention_ratio + target_mlp_ratio > 1.0:
        raise ValueError("attention ratio + mlp ratio must not exceed 1")
    slots = _auto(total_layers_count, target_attention_ratio, target_mlp_ratio)
    if override_pattern is not None:
        forced = _from_pattern(total_layers_count, override_pattern)
        if verbose and any(forced.count(s) != slots.count(s) for s in VALID):
            log.info("override pattern changes the layer mix implied by the ratios")
        slots = forced
    if verbose:
        log.info("hybrid allocation: %s  (%d mamba, %d attention, %d mlp)", "".join(slots),
                 slots.count(MAMBA), slots.count(ATTENTION), slots.count(MLP))
    return slots


if __name__ == "__main__":
    for args in [(56, 0.08, 0.5), (48, 0.08, 0.5), (9, 0.0, 0.0), (9, 0.0, 0.5), (9, 0.3, 0.0)]:
        print(args, "".join(allocate_layers(*args)))
