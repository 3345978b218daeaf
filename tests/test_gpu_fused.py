"""Fused kernels on one GPU (emulated ranks): fp8 wire reduce-scatter against
the bf16 / fp32 result, reduce-scatter + AdamW against torch.optim.AdamW."""
import pytest
import torch

import configurable_hierarchical_allreduce_algorithms_b200 as chb
from configurable_hierarchical_allreduce_algorithms_b200.ops import fused
from configurable_hierarchical_allreduce_algorithms_b200.parallel.comm import Communicator

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("P", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fp8_wire_reduce_scatter(cuda, P, dtype):
    comm = Communicator.emulated(P, scratch_bytes=16 << 20, user_bytes=1 << 20)
    for n in (128, 128 * 37, 128 * 1024):
        g = torch.Generator(device="cuda").manual_seed(n)
        ins = [(torch.rand(n * P, generator=g, device="cuda") * 2 - 1).to(dtype) for _ in range(P)]
        exact = torch.stack([x.double() for x in ins]).sum(0)
        outs = fused.reduce_scatter_fp8(comm, ins, scale=1.0 / P)
        plain = chb.reduce_scatter(comm, ins, algo="radix_batch", scale=1.0 / P)
        for r in range(P):
            want = exact[r * n:(r + 1) * n] / P
            # e4m3 keeps 3 mantissa bits: relative error <= 2^-4 per element of magnitude <= 1
            err = (outs[r].double() - want).abs().max().item()
            assert err < 0.07 * (P - 1) / P + 0.02, err
            rel = (outs[r].double() - want).norm() / want.norm()
            assert rel < 0.05, rel
            # and it stays close to what the full-precision wire gives
            assert (outs[r].double() - plain[r].double()).abs().max().item() < 0.08
    comm.check()
    comm.close()


@pytest.mark.parametrize("P", [1, 2, 4])
def test_reduce_scatter_adam_matches_torch(cuda, P):
    comm = Communicator.emulated(P, scratch_bytes=1 << 20, user_bytes=8 << 20)
    n = 4 * 1031                      # shard length (multiple of 4)
    total = n * P
    g = torch.Generator(device="cuda").manual_seed(3)
    w0 = torch.randn(total, generator=g, device="cuda")
    grads = comm.empty(total, torch.float32)
    grads = grads if isinstance(grads, list) else [grads]
    master = [w0[r * n:(r + 1) * n].clone() for r in range(P)]
    m = [torch.zeros(n, device="cuda") for _ in range(P)]
    v = [torch.zeros(n, device="cuda") for _ in range(P)]
    params = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for _ in range(P)]
    ref_w = torch.nn.Parameter(w0.clone())
    opt = torch.optim.AdamW([ref_w], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in (1, 2, 3):
        per_rank = [torch.randn(total, generator=g, device="cuda") for _ in range(P)]
        for r in range(P):
            grads[r].copy_(per_rank[r])
        fused.reduce_scatter_adam(comm, grads if P > 1 else grads[0], master if P > 1 else master[0],
                                  m if P > 1 else m[0], v if P > 1 else v[0], params if P > 1 else params[0],
                                  lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, step=step,
                                  grad_scale=1.0 / P, use_multimem=False)
        ref_w.grad = torch.stack(per_rank).sum(0) / P
        opt.step()
        got = torch.cat(master)
        torch.testing.assert_close(got, ref_w.detach(), rtol=2e-5, atol=2e-6)
        torch.testing.assert_close(torch.cat(params).float(), ref_w.detach().bfloat16().float(), rtol=1e-2, atol=1e-2)
    comm.check()
    comm.close()


def test_adam_flat_matches_torch(cuda):
    n = 4 * 5003
    g = torch.Generator(device="cuda").manual_seed(5)
    w0 = torch.randn(n, generator=g, device="cuda")
    master, m, v = w0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    pb = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    ref = torch.nn.Parameter(w0.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for step in (1, 2, 3):
        grad = torch.randn(n, generator=g, device="cuda")
        fused.adam_flat(grad, master, m, v, pb, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, step=step)
        ref.grad = grad.clone()
        opt.step()
        torch.testing.assert_close(master, ref.detach(), rtol=2e-5, atol=2e-6)
        torch.testing.assert_close(pb.float(), ref.detach().bfloat16().float(), rtol=1e-2, atol=1e-2)


def test_bucket_fill_casts_overwrites_and_accumulates(cuda):
    """One launch moves a whole bucket's gradients (mixed dtypes, odd lengths, unaligned offsets) into the
    flat fp32 buffer; compared with plain PyTorch fp32 arithmetic."""
    import torch

    from configurable_hierarchical_allreduce_algorithms_b200.ops import fused

    g = torch.Generator(device="cuda").manual_seed(5)
    sizes = [1, 3, 4, 127, 4096, 100003] + [64] * 60          # more tensors than one launch's table holds
    dts = [torch.bfloat16, torch.float32, torch.float16]
    grads = [(torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dts[i % 3]) for i, n in enumerate(sizes)]
    offs, off = [], 0
    for n in sizes:
        offs.append(off)
        off += (n + 3) // 4 * 4 if n != 3 else 3               # one odd offset: the next slot is not 16-byte aligned
    bucket = torch.full((off + 8,), 7.0, device="cuda")
    ref = bucket.clone()
    ow = [i % 2 == 0 for i in range(len(sizes))]
    fused.bucket_fill(bucket, [(gr, o, w) for gr, o, w in zip(grads, offs, ow)])
    for gr, o, w in zip(grads, offs, ow):
        ref[o:o + gr.numel()] = gr.float() if w else ref[o:o + gr.numel()] + gr.float()
    torch.cuda.synchronize()
    assert torch.equal(bucket, ref)
    # a view of a larger gradient (non-zero storage offset) accumulates as well
    big = torch.arange(64, device="cuda", dtype=torch.bfloat16)
    fused.bucket_fill(bucket, [(big[1:33], 0, False)])
    ref[0:32] += big[1:33].float()
    assert torch.equal(bucket, ref)
