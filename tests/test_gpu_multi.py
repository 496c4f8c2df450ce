"""GPU, >= 2 devices: one process per GPU over NCCL - the vocabulary-parallel cross entropy
(its single all-gather) and the sequence-sharded decoder block give the single-GPU result.
Skipped on a single-GPU machine; the same host logic runs on CPU in tests/test_dist_cpu.py."""

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as td

    from custom_cuda_kernals_b200 import dist
    from custom_cuda_kernals_b200.kernels.linear_cross_entropy import linear_cross_entropy
    from custom_cuda_kernals_b200.kernels.matmul_add_bias import matmul_add_bias
    from custom_cuda_kernals_b200.llama_block import LlamaBlock
    from oracle import workloads
    dist.init_from_env(timeout_s=120)
    dev = torch.device("cuda", rank)
    # --- vocabulary-parallel cross entropy: every rank holds whole 128-row tiles of W
    h, w, t = workloads.lce_bf16(tokens=512, hidden=1024, vocab=20000 + 57)
    h, w, t = h.to(dev), w.to(dev), t.to(dev)
    v0, v1 = dist.vocab_range(w.shape[0], rank, world)
    loss = dist.vocab_parallel_linear_cross_entropy(h, w[v0:v1].contiguous(), t, v0)
    rows = dist.vocab_parallel_linear_cross_entropy(h, w[v0:v1].contiguous(), t, v0, reduction="none")
    single = linear_cross_entropy(h, w, t)
    single_rows = linear_cross_entropy(h, w, t, reduction="none")
    # --- vocabulary-parallel gradients: all-reduced d_hidden, own rows of d_weight
    from custom_cuda_kernals_b200.kernels.linear_cross_entropy import linear_cross_entropy_fwd_bwd
    hg, wg, tg = workloads.lce_bf16(tokens=512, hidden=1024, vocab=20480)
    hg, wg, tg = hg.to(dev), wg.to(dev), tg.to(dev)
    g0, g1 = dist.vocab_range(wg.shape[0], rank, world)
    p_loss, p_dh, p_dw = dist.vocab_parallel_linear_cross_entropy_fwd_bwd(hg, wg[g0:g1].contiguous(), tg, g0)
    s_loss, s_dh, s_dw = linear_cross_entropy_fwd_bwd(hg, wg, tg)
    _, p_dh_rows, _ = dist.vocab_parallel_linear_cross_entropy_fwd_bwd(hg, wg[g0:g1].contiguous(), tg, g0, scatter_rows=True)
    r0, r1 = dist.row_range(hg.shape[0], rank, world)
    dh_scale = s_dh.float().abs().max()
    grads_ok = bool(torch.allclose(p_loss, s_loss, rtol=1e-6, atol=1e-6)
                    and (p_dh.float() - s_dh.float()).abs().max() <= 2e-2 * dh_scale
                    and (p_dh_rows.float() - s_dh[r0:r1].float()).abs().max() <= 2e-2 * dh_scale
                    and (p_dw.float() - s_dw[g0:g1].float()).abs().max() <= 2e-2 * s_dw.float().abs().max())
    # --- GEMM column shards written into one output
    a, wt, b = workloads.gemm_bf16(m=512, k=1024, n=2048)
    a, wt, b = a.to(dev), wt.to(dev), b.to(dev)
    n0, n1 = dist.column_range(wt.shape[0], rank, world)
    y_part = matmul_add_bias(a, wt[n0:n1].contiguous(), b[n0:n1].contiguous())
    y_full = matmul_add_bias(a, wt, b)
    # --- decoder block, sequences sharded
    cfg = dict(workloads.LLAMA3_8B, hidden=1024, ffn=2816, n_heads=8, n_kv_heads=2, head_dim=128)
    wd = {k: v.to(dev) for k, v in workloads.block_weights(cfg).items()}
    block = LlamaBlock(wd, 8, 2, cfg["eps"], cfg["theta"], max_seq_len=128)
    x = workloads.block_input(4, 128, 1024).to(dev)
    b0, b1 = dist.sequence_range(4, rank, world)
    with torch.no_grad():
        part = block(x[b0:b1].contiguous())
        full = block(x)
    torch.cuda.synchronize()
    torch.save({"loss": loss.cpu(), "single": single.cpu(), "rows_equal": bool(torch.allclose(rows, single_rows, rtol=1e-6, atol=1e-6)),
                "grads_ok": grads_ok,
                "gemm_equal": bool(torch.equal(y_part, y_full[:, n0:n1])),
                "block_equal": bool(torch.equal(part, full[b0:b1]))}, os.path.join(out_dir, f"r{rank}.pt"))
    td.barrier()
    td.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_two_ranks_match_single_gpu(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    outs = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    for o in outs:
        torch.testing.assert_close(o["loss"], o["single"], rtol=1e-6, atol=1e-6)
        assert o["rows_equal"] and o["gemm_equal"] and o["block_equal"] and o["grads_ok"]
    assert torch.equal(outs[0]["loss"], outs[1]["loss"])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_one_process_drives_two_devices():
    """A single process that uses the library on cuda:0 and then on cuda:1: every launch runs
    on the device that owns its tensors (kernel attributes such as the dynamic shared memory
    limit are per device), and both devices give the same bits."""
    from custom_cuda_kernals_b200 import _native
    from custom_cuda_kernals_b200.kernels.autograd import rmsnorm_residual_backward
    from custom_cuda_kernals_b200.kernels.fp8_quant import fp8_quant
    from custom_cuda_kernals_b200.kernels.linear_cross_entropy import linear_cross_entropy
    from custom_cuda_kernals_b200.kernels.matmul_add_bias import matmul_add_bias
    g = torch.Generator().manual_seed(21)
    x = torch.randn(512, 1024, generator=g).to(torch.bfloat16)
    w = (0.05 * torch.randn(2048, 1024, generator=g)).to(torch.bfloat16)
    small = torch.randn(64, 1024, generator=g).to(torch.bfloat16)
    t = torch.randint(0, 2048, (512,), generator=g)
    outs = []
    for d in (0, 1):
        dev = torch.device("cuda", d)
        xd, wd, sd, td = x.to(dev), w.to(dev), small.to(dev), t.to(dev)
        y = matmul_add_bias(xd, wd)                       # CTA-pair kernel
        ys = matmul_add_bias(sd, wd)                      # narrow-tile kernel
        codes, scale = fp8_quant(xd, "e4m3", "block")     # TMA-staged kernel (dynamic shared memory)
        loss = linear_cross_entropy(xd, wd, td)
        dx, dw = rmsnorm_residual_backward(xd, None, xd, torch.ones(1024, dtype=torch.bfloat16, device=dev), 1e-5)
        assert y.device == dev and _native.take_device_status(y) == 0
        outs.append([o.cpu() for o in (y, ys, codes.view(torch.uint8), scale, loss, dx, dw)])
    for a, b in zip(*outs):
        assert torch.equal(a, b)
