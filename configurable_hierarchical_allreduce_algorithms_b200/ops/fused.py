"""Fused collective + compute kernels: reduce-scatter with an fp8 block-scaled
wire format, and reduce-scatter fused with the sharded AdamW update
(``csrc/kernels/fp8_wire.cu``, ``csrc/kernels/fused_adam.cu``)."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N
from ..parallel.comm import DTYPES, Communicator, _stream_ptr

vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
N.optional("chb_rs_fp8_wire", i32, [vp, i32, C.POINTER(vp), C.POINTER(vp), C.c_longlong, f32, i32, vp])
N.optional("chb_rs_adam", i32, [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp),
                                C.c_longlong, C.POINTER(f32), i32, i32, vp])


N.optional("chb_adam_flat", i32, [vp, vp, vp, vp, vp, C.c_longlong, C.POINTER(f32), vp])
N.optional("chb_bucket_fill", i32, [vp, i32, C.POINTER(vp), C.POINTER(C.c_longlong), C.POINTER(C.c_longlong),
                                    C.POINTER(i32), C.POINTER(C.c_ubyte), vp])


def bucket_fill(bucket: torch.Tensor, items, stream=None):
    """One kernel for a whole gradient bucket: ``items`` = (gradient tensor, element offset in the flat fp32
    ``bucket``, overwrite?) per parameter; bf16 / fp16 / fp32 gradients are cast and either replace their
    slot or are added to it (``csrc/kernels/bucket.cu``)."""
    k = len(items)
    if k == 0:
        return
    assert bucket.dtype == torch.float32 and bucket.is_cuda
    grads = [g if g.is_contiguous() else g.contiguous() for g, _, _ in items]
    src = (vp * k)(*[g.data_ptr() for g in grads])
    off = (C.c_longlong * k)(*[int(o) for _, o, _ in items])
    n = (C.c_longlong * k)(*[g.numel() for g in grads])
    dt = (i32 * k)(*[DTYPES[g.dtype] for g in grads])
    ow = (C.c_ubyte * k)(*[1 if w else 0 for _, _, w in items])
    rc = N.lib().chb_bucket_fill(bucket.data_ptr(), k, src, off, n, dt, ow, _stream_ptr(stream))
    if rc:
        raise RuntimeError(f"chb_bucket_fill failed with code {rc}")


def adam_flat(grad, master, exp_avg, exp_avg_sq, param_bf16, *, lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
              step=1, grad_scale=1.0, stream=None):
    """AdamW on a flat fp32 master tensor fed by a flat fp32 gradient; writes the bf16 parameters."""
    n = master.numel()
    hyper = (f32 * 8)(lr, betas[0], betas[1], eps, weight_decay, 1.0 - betas[0] ** step, 1.0 - betas[1] ** step, grad_scale)
    rc = N.lib().chb_adam_flat(grad.data_ptr(), master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(),
                               param_bf16.data_ptr(), n, hyper, _stream_ptr(stream))
    if rc:
        raise RuntimeError(f"chb_adam_flat failed with code {rc}")


def _lst(x):
    return [x] if isinstance(x, torch.Tensor) else list(x)


def _arr(ts):
    return (vp * len(ts))(*[t.data_ptr() for t in ts])


def reduce_scatter_fp8(comm: Communicator, x, out=None, scale: float = 1.0, nctas: int = 0, stream=None):
    """Sum reduce-scatter whose wire format is fp8 e4m3 in 128-element blocks
    with fp32 scales.  ``x``: P blocks of n elements (n % 128 == 0), f32 or bf16."""
    ins = _lst(x)
    n = ins[0].numel() // comm.P
    outs = _lst(out) if out is not None else [torch.empty(n, dtype=t.dtype, device=t.device) for t in ins]
    rc = N.lib().chb_rs_fp8_wire(comm.handle, DTYPES[ins[0].dtype], _arr(ins), _arr(outs), n, scale, nctas,
                                 _stream_ptr(stream))
    comm._err(rc)
    comm.launches += 1
    return outs if comm.nlocal > 1 else outs[0]


def reduce_scatter_adam(comm: Communicator, grads, master, exp_avg, exp_avg_sq, param_shard, *, lr: float,
                        betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, step: int = 1,
                        grad_scale: float = 1.0, use_multimem: bool | None = None, nctas: int = 0, stream=None):
    """Rank r sums shard r of every rank's flat fp32 gradient buffer (symmetric
    memory), applies AdamW to its fp32 master shard and writes the bf16 shard
    into ``param_shard``.  All tensor arguments: one tensor, or a list of P
    tensors in an emulated world."""
    g, w, m, v, p = _lst(grads), _lst(master), _lst(exp_avg), _lst(exp_avg_sq), _lst(param_shard)
    n = w[0].numel()
    assert g[0].numel() == n * comm.P and g[0].dtype == torch.float32 and p[0].dtype == torch.bfloat16
    if use_multimem is None:
        use_multimem = comm.has_multicast and comm.nlocal == 1 and comm.P > 2
    hyper = (f32 * 8)(lr, betas[0], betas[1], eps, weight_decay, 1.0 - betas[0] ** step, 1.0 - betas[1] ** step,
                      grad_scale)
    rc = N.lib().chb_rs_adam(comm.handle, _arr(g), _arr(w), _arr(m), _arr(v), _arr(p), n, hyper,
                             int(bool(use_multimem)), nctas, _stream_ptr(stream))
    comm._err(rc)
    comm.launches += 1
