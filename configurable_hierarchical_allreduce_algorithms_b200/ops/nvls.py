"""Launcher for the in-switch (NVLS ``multimem``) kernels in ``csrc/kernels/nvls.cu``."""
from __future__ import annotations

import os

from .. import _native as N
from ..parallel.comm import DTYPES, CollectiveError, _stream_ptr

AR_TWO_SHOT, RS, AG, AR_ONE_SHOT = 0, 1, 2, 3
ONE_SHOT_MAX_BYTES = int(os.environ.get("CHB_NVLS_ONESHOT_BYTES", 256 << 10))


def run(comm, coll: str, x, out, count: int, op: str = "sum", scale: float = 1.0, nctas: int = 0, stream=None,
        one_shot: bool | None = None):
    if op != "sum":
        raise CollectiveError(N.ERR_OP, "the multimem kernels implement sums only")
    if coll == "allreduce":
        nbytes = count * x.element_size()
        if one_shot is None:
            one_shot = nbytes <= ONE_SHOT_MAX_BYTES
        mode = AR_ONE_SHOT if one_shot else AR_TWO_SHOT
    elif coll == "reduce_scatter":
        mode = RS
    elif coll == "allgather":
        mode = AG
    else:
        raise CollectiveError(N.ERR_UNSUPPORTED, f"no multimem kernel for {coll}")
    rc = N.lib().chb_nvls_collective(comm.handle, mode, DTYPES[x.dtype], x.data_ptr(), out.data_ptr(), count,
                                     scale, nctas, _stream_ptr(stream))
    comm._err(rc)
    comm.launches += 1
