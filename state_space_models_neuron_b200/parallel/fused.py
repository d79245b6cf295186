"""Switchboard for the fused compute+collective kernels (filled in by parallel/fused_ops)."""
_ENABLED = [True]
_IMPL = [None]


def set_enabled(flag: bool) -> None:
    _ENABLED[0] = bool(flag)


def register(impl) -> None:
    _IMPL[0] = impl


def enabled_for(x) -> bool:
    return bool(_ENABLED[0] and _IMPL[0] is not None and x.is_cuda and _IMPL[0].ready_for(x))


def all_gather_linear(x, weight, bias=None):
    return _IMPL[0].all_gather_linear(x, weight, bias)


def linear_reduce_scatter(x, weight):
    return _IMPL[0].linear_reduce_scatter(x, weight)
