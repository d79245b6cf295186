"""Switchboard for the fused compute+collective kernels (filled in by parallel/fused_ops)."""
import os

_ENABLED = [True]
_IMPL = [None]
# the single-kernel small all-reduce replaces library all-reduces of tiny vectors; SSM_B200_SMALL_AR=0 turns it off
_SMALL_AR = [os.environ.get("SSM_B200_SMALL_AR", "1") != "0"]


_ZERO1 = [os.environ.get("SSM_B200_FUSED_ZERO1", "1") != "0"]
# the two GEMM + collective kernels can be switched off one by one (SSM_B200_FUSED_AG=0 / SSM_B200_FUSED_RS=0 or
# `set_kernel`): the op then runs as the NCCL collective plus the plain GEMM kernel inside the same autograd
# functions, so forward and backward uses switch together and the other fused kernels stay on
_KERNELS = {"ag_gemm": os.environ.get("SSM_B200_FUSED_AG", "1") != "0",
            "gemm_rs": os.environ.get("SSM_B200_FUSED_RS", "1") != "0"}


def is_enabled() -> bool:
    return bool(_ENABLED[0])


def zero1_enabled() -> bool:
    return bool(_ZERO1[0])


def set_enabled(flag: bool) -> None:
    _ENABLED[0] = bool(flag)


def set_kernel(name: str, flag: bool) -> None:
    if name not in _KERNELS:
        raise KeyError(f"unknown fused kernel {name!r}; known: {sorted(_KERNELS)}")
    _KERNELS[name] = bool(flag)


def kernel_enabled(name: str) -> bool:
    return bool(_KERNELS[name])


def kernels() -> dict:
    return dict(_KERNELS)


def register(impl) -> None:
    _IMPL[0] = impl


def enabled_for(x) -> bool:
    if not (_ENABLED[0] and x.is_cuda):
        return False
    if _IMPL[0] is None:
        from . import fused_ops
        fused_ops.install()
    return bool(_IMPL[0].ready_for(x))


def all_gather_linear(x, weight, bias=None, ce=None):
    """`ce` = (labels, vocab_start): also return the cross-entropy statistics of the output rows, `(y, stats)`."""
    return _IMPL[0].all_gather_linear(x, weight, bias, ce)


def all_gather_multi_linear(x, weights):
    """Outputs of several column-parallel weights behind one fused sequence all-gather, or None."""
    return _IMPL[0].all_gather_multi_linear(x, list(weights))


def linear_reduce_scatter(x, weight):
    return _IMPL[0].linear_reduce_scatter(x, weight)


def small_allreduce(data, op: str = "sum") -> bool:
    """Fused small all-reduce over the TP group; False means "not available, use the library collective"."""
    if not (_ENABLED[0] and _SMALL_AR[0] and data.is_cuda) or _IMPL[0] is None:
        return False
    from . import fused_ops
    return fused_ops.small_allreduce(data, op)


def vocab_embed_scatter(ids, weight, vocab_start: int):
    """Fused vocabulary-parallel embedding with sequence-parallel output; None means "use the library path"."""
    if not (_ENABLED[0] and weight.is_cuda):
        return None
    if _IMPL[0] is None:
        from . import fused_ops
        fused_ops.install()
    from . import fused_ops
    return fused_ops.vocab_embed_scatter(ids, weight, vocab_start)


def allreduce_bf16(x):
    """One-kernel all-reduce of a bf16 activation outside autograd (decode); None means "use the library"."""
    if not (_ENABLED[0] and x.is_cuda):
        return None
    if _IMPL[0] is None:
        from . import fused_ops
        fused_ops.install()
    from . import fused_ops
    return fused_ops.allreduce_bf16(x)
