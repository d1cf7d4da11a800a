"""Expert parallelism on 2 GPUs (skipped with fewer): every rank routes its own tokens, rows
travel to the owning rank over NCCL and back. Each rank's outputs and gradients must equal the
oracle's for the concatenated batch: routing is per token, expert outputs are per row, the
statistics, the aux/z normalisation and the router gradient are over all ranks' tokens."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q, transport, gemm_impl=3, waves=1, shape=(900, 256, 384, 8, 2)):
    try:
        sys.path[:0] = [ROOT, os.path.join(ROOT, "test-model-thing-cuda_b200"), os.path.join(ROOT, "tests")]
        # waves > 10: tens = expert waves, units = how many of them the second stream fetches (the rest: final combine)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), TMT_MOE_EP_WAVES=str(waves // 10 if waves > 10 else waves))
        if waves > 10:
            os.environ["TMT_MOE_EP_FETCH"] = str(waves % 10)
        import torch.distributed as dist
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        from tmt_moe_b200 import synth
        import gpu_util as G
        import tmt_moe_b200 as M
        from oracle import oracle as O
        T, D, H, E, K = shape
        rf = True
        data = [synth.make(T, D, H, E, K, rf, seed=70 + g, w_std=0.06, router_std=0.1, dy_std=0.05) for g in range(world)]
        allX = np.concatenate([d["X"] for d in data])
        alldY = np.concatenate([d["dY"] for d in data])
        base = data[0]                       # weights of rank 0's generator are THE weights (replicated router)
        ref = O.forward(allX, base["Wr"], base["Wup"], base["Wdown"], K)
        rb = O.backward(ref, alldY, 0.1, 0.001)
        EL = E // world
        mine = dict(base, X=data[rank]["X"], dY=data[rank]["dY"],
                    Wup=base["Wup"][rank * EL:(rank + 1) * EL], Wdown=base["Wdown"][rank * EL:(rank + 1) * EL])
        moe = M.MoE(T, D, E, K, hidden=H, router_dtype=M.F32, training=True, device=rank, ep_world=world, ep_rank=rank,
                    ep_capacity_factor=2.0, ep_transport=transport, gemm_impl=gemm_impl, host_io=True)
        moe.ep_init_torch(dist)
        X, dY, Wr = G.dev(mine["X"]), G.dev(mine["dY"]), G.dev(mine["Wr"])
        Wup_all, Wdown_all = G.dev(mine["Wup"]), G.dev(mine["Wdown"])
        Wup, Wdown = [Wup_all[e] for e in range(EL)], [Wdown_all[e] for e in range(EL)]
        Y = torch.zeros((T, D), dtype=torch.int16, device="cuda")
        dX = torch.zeros((T, D), dtype=torch.int16, device="cuda")
        dWr = torch.full((E, D), float("nan"), device="cuda")
        dWup_all = torch.full(tuple(Wup_all.shape), float("nan"), device="cuda")
        dWdown_all = torch.full(tuple(Wdown_all.shape), float("nan"), device="cuda")
        for it in range(2):                  # twice: the second step reuses every buffer
            moe.forward(X, Wr, Wup, Wdown, Y, 0.0)
            moe.backward(dY, Wr, Wup, Wdown, dWr, [dWup_all[e] for e in range(EL)], [dWdown_all[e] for e in range(EL)],
                         dX, 0.1, 0.001)
            torch.cuda.synchronize()
        assert moe.device_status() == 0
        sl = slice(rank * T, (rank + 1) * T)
        np.testing.assert_array_equal(moe.read("idx"), ref["idx"][sl])
        np.testing.assert_array_equal(moe.read("logits").view(np.uint32), ref["logits"][sl].view(np.uint32))
        stat, counts, aux = moe.stats()
        np.testing.assert_array_equal(counts, ref["counts"])
        np.testing.assert_allclose(stat, ref["stat"], rtol=1e-4, atol=1e-6)
        assert abs(aux - ref["aux"]) <= 1e-4 * abs(ref["aux"])
        errs = {
            "Y": synth.rel_l2(O.bf16_to_f32(G.host_u16(Y)), O.bf16_to_f32(ref["Y"][sl])),
            "dX": synth.rel_l2(O.bf16_to_f32(G.host_u16(dX)), O.bf16_to_f32(rb["dX"][sl])),
            "dWr": synth.rel_l2(dWr.cpu().numpy(), rb["dWr"]),
            "dWup": synth.rel_l2(dWup_all.cpu().numpy(), rb["dWup"][rank * EL:(rank + 1) * EL]),
            "dWdown": synth.rel_l2(dWdown_all.cpu().numpy(), rb["dWdown"][rank * EL:(rank + 1) * EL]),
        }
        assert errs["Y"] <= 1e-2 and max(errs.values()) <= 3e-2, errs
        # the host-buffer step (pinned X / dY in, Y / dX / statistics out) gives exactly the device-pointer results
        pin = lambda a: torch.from_numpy(a.view(np.int16).copy()).pin_memory()
        hX, hdY = pin(mine["X"]), pin(mine["dY"])
        hY, hdX = torch.zeros_like(hX).pin_memory(), torch.zeros_like(hX).pin_memory()
        hstat = torch.zeros(E + 1).pin_memory()
        dWr2 = torch.zeros_like(dWr)
        for it in range(2):
            moe.step_host(hX, hdY, Wr, Wup, Wdown, dWr2, [dWup_all[e] for e in range(EL)], [dWdown_all[e] for e in range(EL)],
                          hY, hdX, hstat, 0.0, 0.1, 0.001, wait=(it == 1))
        assert moe.device_status() == 0
        np.testing.assert_array_equal(hY.numpy().view(np.uint16), G.host_u16(Y))
        np.testing.assert_array_equal(hdX.numpy().view(np.uint16), G.host_u16(dX))
        np.testing.assert_array_equal(dWr2.cpu().numpy(), dWr.cpu().numpy())
        np.testing.assert_allclose(hstat.numpy()[:E], ref["stat"][:E], rtol=1e-4, atol=1e-6)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok %s" % {k: "%.1e" % v for k, v in errs.items()}))
    except Exception as exc:  # noqa: BLE001
        import traceback
        q.put((rank, "FAIL: %s\n%s" % (exc, traceback.format_exc())))


SMALL = (900, 256, 384, 8, 2)
C5_WIDTHS = (1024, 2048, 2048, 64, 4)      # the benchmarked configuration's widths, 32 experts per rank, on a token sample


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("transport,gemm_impl,waves,shape", [
    pytest.param(0, 3, 1, SMALL, id="peer"), pytest.param(1, 3, 1, SMALL, id="nccl"),
    pytest.param(0, 2, 1, SMALL, id="peer-cta_pairs"), pytest.param(1, 2, 1, SMALL, id="nccl-cta_pairs"),
    pytest.param(0, 2, 2, SMALL, id="peer-cta_pairs-two_expert_waves"),
    pytest.param(0, 2, 4, SMALL, id="peer-cta_pairs-four_expert_waves"),
    pytest.param(0, 0, 1, C5_WIDTHS, id="peer-config5_widths"), pytest.param(1, 0, 1, C5_WIDTHS, id="nccl-config5_widths"),
    pytest.param(0, 0, 4, C5_WIDTHS, id="peer-config5_widths-four_expert_waves"),
    pytest.param(0, 0, 42, C5_WIDTHS, id="peer-config5_widths-four_expert_waves-two_fetched"),
    pytest.param(0, 2, 40, SMALL, id="peer-cta_pairs-four_expert_waves-none_fetched"),
    pytest.param(2, 2, 1, SMALL, id="dma-cta_pairs-one_wave"), pytest.param(2, 2, 4, SMALL, id="dma-cta_pairs-four_expert_waves"),
    pytest.param(2, 3, 2, SMALL, id="dma-two_expert_waves"), pytest.param(2, 0, 4, C5_WIDTHS, id="dma-config5_widths")])
def test_expert_parallel_two_gpus(transport, gemm_impl, waves, shape):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 200 + 7 * transport + 17 * gemm_impl + 3 * waves + (60 if shape[1] > 256 else 0)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, transport, gemm_impl, waves, shape)) for r in range(world)]
    for p in procs:
        p.start()
    res = []
    try:
        for _ in procs:
            res.append(q.get(timeout=600))
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    for rank, msg in res:
        assert msg.startswith("ok"), "rank %d: %s" % (rank, msg)
    assert len(res) == world
