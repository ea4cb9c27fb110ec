"""Expert-parallel grouped GEMM over NCCL (needs >= 2 GPUs; skipped otherwise): the result of
dispatch -> local grouped GEMM -> combine on every rank equals the single-GPU grouped GEMM over
all experts, and dW of the local experts equals the corresponding slice."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    for p in (str(root), str(root / "transformers-qwen3-moe-fused_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from qwen3_moe_fused.grouped_gemm.backward_dw import grouped_gemm_backward_dw
        from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
        from qwen3_moe_fused.kernels.indexing import get_expert_counts_and_idx
        from qwen3_moe_fused.parallel_ep import ExpertParallelPlan

        E, K, N, rows = 16, 256, 384, 3000
        e_local = E // world
        gw = torch.Generator().manual_seed(7)
        w_all = (torch.randn(E, N, K, generator=gw) * 0.05).to(torch.bfloat16)
        g = torch.Generator().manual_seed(100 + rank)
        ids = torch.randint(0, E, (rows,), generator=g)
        ids[ids == 3] = 2  # expert 3 receives nothing from anybody
        x = torch.randn(rows, K, generator=g).to(torch.bfloat16)
        dy = torch.randn(rows, N, generator=g).to(torch.bfloat16)
        counts, inv_idx, idx = get_expert_counts_and_idx(ids.to(dev), E)
        xs = x.to(dev)[inv_idx.long()].contiguous()
        dys = dy.to(dev)[inv_idx.long()].contiguous()
        w_local = w_all[rank * e_local:(rank + 1) * e_local].to(dev).contiguous()

        plan = ExpertParallelPlan.build(counts, world, rank, dev)
        x_loc = plan.dispatch(xs)
        y = plan.combine(plan.grouped(grouped_gemm_forward, x_loc, w_local))
        dw = plan.grouped_dw(grouped_gemm_backward_dw, x_loc, plan.dispatch(dys), torch.bfloat16, e_local)
        # single-GPU reference over all experts on this rank's own rows
        y_ref = grouped_gemm_forward(xs, w_all.to(dev), counts)
        torch.cuda.synchronize()
        err = float((y.float() - y_ref.float()).abs().max() / y_ref.float().abs().max())
        assert err < 1e-2, f"rank {rank}: forward mismatch {err}"
        torch.save({"xs": xs.cpu(), "dys": dys.cpu(), "ids": ids[inv_idx.cpu().long()], "dw": dw.cpu()}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_matches_single_gpu(tmp_path):
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    from oracle import moe_oracle as O

    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    saved = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    E, e_local = 16, 8
    xs = torch.cat([s["xs"] for s in saved]).float().numpy()
    dys = torch.cat([s["dys"] for s in saved]).float().numpy()
    ids = torch.cat([s["ids"] for s in saved]).numpy()
    for r in range(world):
        for le in range(e_local):
            e = r * e_local + le
            sel = ids == e
            ref = dys[sel].T @ xs[sel]
            got = saved[r]["dw"][le].float().numpy()
            assert O.rel_err(got, ref) < 1e-2 if sel.any() else not got.any(), f"dW of expert {e}"


def _peer_worker(rank, world, port, out_dir):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    for p in (str(root), str(root / "transformers-qwen3-moe-fused_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from qwen3_moe_fused import _lib
        from qwen3_moe_fused.grouped_gemm.backward_dw import grouped_gemm_backward_dw
        from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
        from qwen3_moe_fused.grouped_gemm.forward_transposed import grouped_gemm_forward_transposed
        from qwen3_moe_fused.kernels.indexing import get_expert_counts_and_idx
        from qwen3_moe_fused.parallel_ep import PeerChannel, PeerPlan, peer_fence, peer_grouped_gemm, peer_push

        E, K, N, rows = 16, 256, 384, 3000
        bf = torch.bfloat16
        e_local = E // world
        gw = torch.Generator().manual_seed(7)
        w_all = (torch.randn(E, N, K, generator=gw) * 0.05).to(bf)
        g = torch.Generator().manual_seed(100 + rank)
        ids = torch.randint(0, E, (rows,), generator=g)
        ids[ids == 3] = 2  # expert 3 receives nothing from anybody
        x = torch.randn(rows, K, generator=g).to(bf)
        dy = torch.randn(rows, N, generator=g).to(bf)
        counts, inv_idx, idx = get_expert_counts_and_idx(ids.to(dev), E)
        xs = x.to(dev)[inv_idx.long()].contiguous()
        dys = dy.to(dev)[inv_idx.long()].contiguous()
        w_local = w_all[rank * e_local:(rank + 1) * e_local].to(dev).contiguous()

        plan = PeerPlan.build(counts, world, rank)
        cap = rows * world
        ch_x, ch_dy = PeerChannel(cap, K, bf, dev), PeerChannel(cap, N, bf, dev)
        ch_y, ch_dx = PeerChannel(rows, N, bf, dev), PeerChannel(rows, K, bf, dev)
        ch_y.local.fill_(9.0)
        ch_dx.local.fill_(9.0)
        token = torch.zeros(1, device=dev)
        peer_fence(token)                       # every rank's buffers exist and are initialised
        peer_push(plan, xs, ch_x)
        peer_push(plan, dys, ch_dy)
        peer_fence(token)                       # every rank's rows have arrived
        peer_grouped_gemm(plan, ch_x, w_local, ch_y)
        peer_grouped_gemm(plan, ch_dy, w_local, ch_dx, transposed=True)
        dw = grouped_gemm_backward_dw(ch_x.local, ch_dy.local, plan.local_m_sizes, bf)
        peer_fence(token)                       # every rank's results have arrived
        torch.cuda.synchronize()
        assert _lib.read_error_flag() == 0
        y_ref = grouped_gemm_forward(xs, w_all.to(dev), counts)
        dx_ref = grouped_gemm_forward_transposed(dys, w_all.to(dev), counts)
        torch.cuda.synchronize()
        for name, got, ref in (("y", ch_y.local, y_ref), ("dx", ch_dx.local, dx_ref)):
            err = float((got.float() - ref.float()).abs().max() / ref.float().abs().max())
            assert err < 1e-2, f"rank {rank}: {name} mismatch {err}"
        torch.save({"xs": xs.cpu(), "dys": dys.cpu(), "ids": ids[inv_idx.cpu().long()], "dw": dw.cpu(),
                    "exact": bool(torch.equal(ch_y.local, y_ref) and torch.equal(ch_dx.local, dx_ref))},
                   os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_peer_memory_expert_parallel_matches_single_gpu(tmp_path):
    """Row push over peer memory + forward / dX with TMA stores into the source rank's memory."""
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    from oracle import moe_oracle as O

    mp.spawn(_peer_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    saved = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    E, e_local = 16, 8
    xs = torch.cat([s["xs"] for s in saved]).float().numpy()
    dys = torch.cat([s["dys"] for s in saved]).float().numpy()
    ids = torch.cat([s["ids"] for s in saved]).numpy()
    for r in range(world):
        for le in range(e_local):
            e = r * e_local + le
            sel = ids == e
            ref = dys[sel].T @ xs[sel]
            got = saved[r]["dw"][le].float().numpy()
            assert O.rel_err(got, ref) < 1e-2 if sel.any() else not got.any(), f"dW of expert {e}"


def _block_worker(rank, world, port, out_dir):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    for p in (str(root), str(root / "transformers-qwen3-moe-fused_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from qwen3_moe_fused import _lib
        from qwen3_moe_fused.moe_block import moe_block_forward
        from qwen3_moe_fused.parallel_ep import PeerMoeBlock

        E, H, I, T, k = 16, 256, 192, 1000, 4
        bf = torch.bfloat16
        e_local = E // world
        gw = torch.Generator().manual_seed(11)
        mk = lambda *shape, sc: (torch.randn(*shape, generator=gw) * sc).to(bf).to(dev)
        gate_w, gate_p, up_p, down_p = mk(E, H, sc=0.05), mk(E, I, H, sc=0.05), mk(E, I, H, sc=0.05), mk(E, H, I, sc=0.05)
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(200 + rank)).to(bf).to(dev)
        lo, hi = rank * e_local, (rank + 1) * e_local
        with torch.no_grad():
            ref, ref_logits = moe_block_forward(x.view(1, T, H), gate_w, gate_p, up_p, down_p, k, True)
        outs = []
        # token-deduplicated dispatch (default capacity: every routing fits), then one row per (token, expert)
        for kwargs in (dict(max_tokens=T), dict(capacity_factor=2.0)):
            block = PeerMoeBlock(world, rank, dev, H, T * k, bf, **kwargs)
            for _ in range(2):  # the second call reuses the buffers
                out, logits = block.forward(x, gate_w, gate_p[lo:hi].contiguous(), up_p[lo:hi].contiguous(),
                                            down_p[lo:hi].contiguous(), k, True)
            torch.cuda.synchronize()
            block.check()
            assert _lib.read_error_flag() == 0
            err = float((out.float() - ref.view(T, H).float()).abs().max() / ref.float().abs().max())
            assert torch.equal(logits, ref_logits) and err < 1e-2, f"rank {rank}: block mismatch {err} ({kwargs})"
            outs.append(out)
        assert torch.equal(outs[0], outs[1]), "both dispatches deliver the same rows, so the outputs are identical"
        # a receive buffer that is too small: rows are dropped, never written out of bounds, and the next call raises
        from qwen3_moe_fused.parallel_ep import ReceiveOverflow

        small = PeerMoeBlock(world, rank, dev, H, T * k, bf, capacity_factor=0.25, max_tokens=T)
        small.forward(x, gate_w, gate_p[lo:hi].contiguous(), up_p[lo:hi].contiguous(), down_p[lo:hi].contiguous(), k, True)
        raised = False
        try:
            small.forward(x, gate_w, gate_p[lo:hi].contiguous(), up_p[lo:hi].contiguous(), down_p[lo:hi].contiguous(), k, True)
        except ReceiveOverflow:
            raised = True
        flags = torch.tensor([int(raised)], device=dev)
        dist.all_reduce(flags)
        assert int(flags) >= 1, "no rank noticed that rows had been dropped"
        torch.cuda.synchronize()
        assert _lib.read_error_flag() == 0
    finally:
        dist.destroy_process_group()


def test_peer_memory_block_forward_matches_single_gpu(tmp_path):
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_block_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
