"""Switchboard for the fused compute+collective kernels (filled in by parallel/fused_ops)."""
_ENABLED = [True]
_IMPL = [None]


def set_enabled(flag: bool) -> None:
    _ENABLED[0] = bool(flag)


def register(impl) -> None:
    _IMPL[0] = impl


def enabled_for(x) -> bool:
    if not (_ENABLED[0] and x.is_cuda):
        return False
    if _IMPL[0] is None:
        from . import fused_ops
        fused_ops.install()
    return bool(_IMPL[0].ready_for(x))


def all_gather_linear(x, weight, bias=None):
    return _IMPL[0].all_gather_linear(x, weight, bias)


def linear_reduce_scatter(x, weight):
    return _IMPL[0].linear_reduce_scatter(x, weight)
