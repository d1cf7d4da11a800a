"""Expert-parallel host logic on CPU ranks: two gloo processes route their own tokens with the
oracle, exchange per-expert counts, compute the exchange plan with the library's own
tmt_moe_ep_plan and move rows with point-to-point messages in exactly the order the CUDA path
posts its NCCL sends and receives. The rows that arrive in each expert group must be the rows a
single process would have grouped, and the way back must restore every token-side slot."""
import ctypes
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PAD = 128


def _plan(lib, G, r, E, cnt_all):
    EL = E // G
    tok_poff = np.zeros(E + 1, np.int32)
    x_counts = np.zeros(EL, np.int32)
    x_poff = np.zeros(EL + 1, np.int32)
    src_off = np.zeros(G * EL, np.int32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    rows = lib.tmt_moe_ep_plan(G, r, E, PAD, p(np.ascontiguousarray(cnt_all, np.int32)), p(tok_poff), p(x_counts),
                               p(x_poff), p(src_off))
    return rows, tok_poff, x_counts, x_poff, src_off.reshape(G, EL)


def _exchange(to_experts, src, dst, G, r, E, cnt_all, tok_poff, x_poff, src_off):
    """Same loop as exchange() in csrc/ep.cu, with gloo isend / irecv (gloo has no message to
    oneself, so the rank's own rows are copied; NCCL handles that pair like any other)."""
    EL = E // G
    ops = []
    for g in range(G):
        for le in range(EL):
            e = g * EL + le
            n_tok = int(cnt_all[r, e])
            n_exp = int(cnt_all[g, r * EL + le])
            tok_row = int(tok_poff[e])
            exp_row = int(x_poff[le] + src_off[g, le])
            if g == r:
                if to_experts:
                    dst[exp_row:exp_row + n_exp] = src[tok_row:tok_row + n_tok]
                else:
                    dst[tok_row:tok_row + n_tok] = src[exp_row:exp_row + n_exp]
                continue
            if to_experts:
                if n_tok:
                    ops.append(dist.P2POp(dist.isend, src[tok_row:tok_row + n_tok].contiguous(), g))
                if n_exp:
                    ops.append(dist.P2POp(dist.irecv, dst[exp_row:exp_row + n_exp], g))
            else:
                if n_exp:
                    ops.append(dist.P2POp(dist.isend, src[exp_row:exp_row + n_exp].contiguous(), g))
                if n_tok:
                    ops.append(dist.P2POp(dist.irecv, dst[tok_row:tok_row + n_tok], g))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()


def _worker(rank, world, port, q):
    sys.path[:0] = [ROOT, os.path.join(ROOT, "test-model-thing-cuda_b200"), os.path.join(ROOT, "tests")]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tmt_moe_b200 import synth
        import tmt_moe_b200 as M
        from oracle import oracle as O
        lib = M.load()
        T, D, E, K = 200, 64, 6, 2
        data = [synth.make(T, D, 0, E, K, seed=50 + g, router_std=0.3) for g in range(world)]
        for d in data:
            d["Wr"] = data[0]["Wr"]                     # replicated router
        mine = data[rank]
        rt = O.router(mine["X"], mine["Wr"], K)
        counts, off, poff, slot_of = O.layout(rt["idx"], E, PAD)
        gathered = [torch.zeros(E, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(counts.astype(np.int32)))
        cnt_all = torch.stack(gathered).numpy()
        rows, tok_poff, x_counts, x_poff, src_off = _plan(lib, world, rank, E, cnt_all)
        assert (tok_poff == poff).all()                  # the plan's token-side layout is the single-GPU layout
        EL = E // world
        assert rows == x_poff[EL] and (x_poff % PAD == 0).all()
        # token-side grouped rows: value = (global token id, column) so that arrivals can be identified
        Xs = torch.zeros((int(poff[E]), 4), dtype=torch.float32)
        for t in range(T):
            for j in range(K):
                Xs[slot_of[t, j]] = torch.tensor([rank, t, j, rt["idx"][t, j]], dtype=torch.float32)
        Xg = torch.full((int(rows), 4), -1.0)
        _exchange(True, Xs, Xg, world, rank, E, cnt_all, tok_poff, x_poff, src_off)
        # expectation from a single process that sees every rank's routing
        for le in range(EL):
            e = rank * EL + le
            want = []
            for g in range(world):
                rg = O.router(data[g]["X"], data[g]["Wr"], K)
                for t in range(T):
                    for j in range(K):
                        if rg["idx"][t, j] == e:
                            want.append([g, t, j, e])
            got = Xg[x_poff[le]:x_poff[le] + x_counts[le]].numpy()
            assert x_counts[le] == len(want)
            np.testing.assert_array_equal(got, np.array(want, np.float32).reshape(-1, 4))
            assert (Xg[x_poff[le] + x_counts[le]:x_poff[le + 1]] == -1).all()    # pad rows untouched
        # the way back restores every slot
        back = torch.full_like(Xs, -2.0)
        _exchange(False, Xg * 2, back, world, rank, E, cnt_all, tok_poff, x_poff, src_off)
        for t in range(T):
            for j in range(K):
                np.testing.assert_array_equal(back[slot_of[t, j]].numpy(), 2 * Xs[slot_of[t, j]].numpy())
        q.put((rank, "ok"))
    except Exception as exc:  # noqa: BLE001
        import traceback
        q.put((rank, "FAIL: %s\n%s" % (exc, traceback.format_exc())))
    finally:
        dist.destroy_process_group()


def test_plan_rejects_bad_arguments():
    sys.path[:0] = [os.path.join(ROOT, "test-model-thing-cuda_b200")]
    import tmt_moe_b200 as M
    lib = M.load()
    z = np.zeros(16, np.int32)
    p = z.ctypes.data_as(ctypes.c_void_p)
    assert lib.tmt_moe_ep_plan(2, 0, 5, 128, p, p, p, p, p) == -1     # experts not divisible by ranks
    assert lib.tmt_moe_ep_plan(2, 2, 4, 128, p, p, p, p, p) == -1     # rank out of range


def _overflow_worker(rank, world, port, q):
    """Every rank routes its own tokens with a bias that sends almost everything to rank 0's experts, gathers the
    counts and runs the library's capacity check: all ranks must name the same overloaded rank and row count."""
    sys.path[:0] = [ROOT, os.path.join(ROOT, "test-model-thing-cuda_b200"), os.path.join(ROOT, "tests")]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tmt_moe_b200 import synth
        import tmt_moe_b200 as M
        from oracle import oracle as O
        lib = M.load()
        T, D, E, K = 256, 64, 6, 2
        d = synth.make(T, D, 0, E, K, seed=90 + rank, router_std=0.3)
        d["Wr"] = synth.make(T, D, 0, E, K, seed=90, router_std=0.3)["Wr"]
        bias = np.array([40, 40] + [0] * (E - 2), np.float32)        # experts 0 and 1 (rank 0 at any world size here) take every token
        rt = O.router(d["X"], d["Wr"], K, bias=bias)
        counts = O.layout(rt["idx"], E, PAD)[0]
        gathered = [torch.zeros(E, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(counts.astype(np.int32)))
        cnt_all = np.ascontiguousarray(torch.stack(gathered).numpy(), np.int32)
        p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        # the capacity of a handle created with ep_capacity_factor = 1.0: roundup(T*K, pad) + pad * local experts
        EL = E // world
        x_cap = (T * K + PAD - 1) // PAD * PAD + PAD * EL
        rows = ctypes.c_longlong(-1)
        bad = lib.tmt_moe_ep_check_capacity(world, E, PAD, p(cnt_all), ctypes.c_longlong(x_cap), ctypes.byref(rows))
        roomy = lib.tmt_moe_ep_check_capacity(world, E, PAD, p(cnt_all), ctypes.c_longlong(world * T * K + PAD * EL), None)
        q.put((rank, "ok", int(bad), int(rows.value), int(roomy)))
    except Exception as exc:  # noqa: BLE001
        import traceback
        q.put((rank, "FAIL: %s\n%s" % (exc, traceback.format_exc()), 0, 0, 0))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_capacity_overflow_is_seen_by_every_rank(world):
    """A step that routes more rows to one rank than it has room for: every rank reaches the same verdict from the
    gathered counts (with either transport the step is refused everywhere, before any row moves)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29100 + os.getpid() % 400 + world
    procs = [ctx.Process(target=_overflow_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg, bad, rows, roomy in res:
        assert msg == "ok", "rank %d: %s" % (rank, msg)
    verdicts = {(bad, rows, roomy) for _, _, bad, rows, roomy in res}
    assert len(verdicts) == 1, res                      # the same on every rank
    bad, rows, roomy = verdicts.pop()
    assert bad == 0 and rows == world * 256 * 2 and roomy == -1     # everything went to rank 0's two experts (multiples of 128)


def test_capacity_check_arguments():
    sys.path[:0] = [os.path.join(ROOT, "test-model-thing-cuda_b200")]
    import tmt_moe_b200 as M
    lib = M.load()
    cnt = np.array([[130, 0, 1, 0], [0, 0, 0, 300]], np.int32)       # 2 ranks, 4 experts
    p = cnt.ctypes.data_as(ctypes.c_void_p)
    rows = ctypes.c_longlong(0)
    assert lib.tmt_moe_ep_check_capacity(2, 4, 128, p, ctypes.c_longlong(256), ctypes.byref(rows)) == 1
    assert rows.value == 128 + 384                      # rank 1: expert 2 has 1 row -> 128, expert 3 has 300 -> 384
    assert lib.tmt_moe_ep_check_capacity(2, 4, 128, p, ctypes.c_longlong(512), None) == -1
    assert lib.tmt_moe_ep_check_capacity(2, 4, 128, p, ctypes.c_longlong(255), ctypes.byref(rows)) == 0 and rows.value == 256
    assert lib.tmt_moe_ep_check_capacity(2, 5, 128, p, ctypes.c_longlong(512), None) == -2


@pytest.mark.parametrize("world", [2, 3])
def test_exchange_plan_two_cpu_ranks(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 400 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in res:
        assert msg == "ok", "rank %d: %s" % (rank, msg)


@pytest.mark.gpu
@pytest.mark.parametrize("G,E,pad", [(8, 64, 256), (2, 8, 128), (4, 64, 256), (8, 8, 128), (3, 6, 128)])
def test_device_plan_kernel_equals_the_host_plan(G, E, pad):
    """The plan kernel of the peer transport (no host synchronisation in a step) against tmt_moe_ep_plan for every rank,
    on one GPU, including the 8-rank layout of the benchmarked configuration; then an overflow: status 4 on every
    rank, tables clamped to the capacity."""
    sys.path[:0] = [os.path.join(ROOT, "test-model-thing-cuda_b200")]
    import tmt_moe_b200 as M
    lib = M.load()
    rng = np.random.default_rng(G * 1000 + E)
    EL = E // G
    cnt_all = rng.integers(0, 900, size=(G, E)).astype(np.int32)
    cnt_all[:, rng.integers(0, E)] = 0                      # an expert nobody routes to
    cnt_all[rng.integers(0, G), :] += 3
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    totals = []
    for r in range(G):
        tok_poff = np.zeros(E + 1, np.int32); x_counts = np.zeros(EL, np.int32)
        x_poff = np.zeros(EL + 1, np.int32); src_off = np.zeros(G * EL, np.int32)
        rows = lib.tmt_moe_ep_plan(G, r, E, pad, p(cnt_all), p(tok_poff), p(x_counts), p(x_poff), p(src_off))
        totals.append(rows)
    x_cap = int(max(totals)) + 2 * pad
    for r in range(G):
        tok_poff = np.zeros(E + 1, np.int32); x_counts = np.zeros(EL, np.int32)
        x_poff = np.zeros(EL + 1, np.int32); src_off = np.zeros(G * EL, np.int32)
        rows = lib.tmt_moe_ep_plan(G, r, E, pad, p(cnt_all), p(tok_poff), p(x_counts), p(x_poff), p(src_off))
        tables = np.full(2 * EL + 2 + x_cap // 128, 7, np.int32)
        dest = np.zeros(E, np.int32); world = np.zeros(E, np.int32); status = np.zeros(1, np.int32)
        rc = lib.tmt_moe_ep_plan_device(G, r, E, pad, x_cap, p(cnt_all), p(tables), p(dest), p(world), p(status))
        assert rc == 0, lib.tmt_moe_last_error().decode()
        assert status[0] == 0
        np.testing.assert_array_equal(tables[:EL + 1], x_poff)
        np.testing.assert_array_equal(tables[EL + 1:2 * EL + 1], x_counts)
        assert tables[2 * EL + 1] == rows // 128
        te = tables[2 * EL + 2:]
        want_te = np.full(x_cap // 128, -1, np.int32)
        for le in range(EL):
            want_te[x_poff[le] // 128:x_poff[le + 1] // 128] = le
        np.testing.assert_array_equal(te, want_te)
        np.testing.assert_array_equal(world, cnt_all.sum(0))
        # where this rank's rows start inside each owner's group: the owner's plan
        for g in range(G):
            o_tok = np.zeros(E + 1, np.int32); o_cnt = np.zeros(EL, np.int32)
            o_poff = np.zeros(EL + 1, np.int32); o_src = np.zeros(G * EL, np.int32)
            lib.tmt_moe_ep_plan(G, g, E, pad, p(cnt_all), p(o_tok), p(o_cnt), p(o_poff), p(o_src))
            np.testing.assert_array_equal(dest[g * EL:(g + 1) * EL], o_poff[:EL] + o_src.reshape(G, EL)[r])
    # a capacity below the fullest rank: every rank reports it, and no table points past the capacity
    small = (int(max(totals)) // pad - 1) * pad
    for r in range(G):
        tables = np.zeros(2 * EL + 2 + small // 128, np.int32)
        dest = np.zeros(E, np.int32); world = np.zeros(E, np.int32); status = np.zeros(1, np.int32)
        assert lib.tmt_moe_ep_plan_device(G, r, E, pad, small, p(cnt_all), p(tables), p(dest), p(world), p(status)) == 0
        assert status[0] == 4
        assert tables[:EL + 1].max() <= small and tables[2 * EL + 1] <= small // 128


@pytest.mark.parametrize("G,E,pad,W", [(8, 64, 256, 4), (4, 64, 256, 4), (2, 64, 256, 4), (2, 8, 128, 4), (8, 16, 128, 4), (3, 6, 128, 2)])
def test_plan_invariants_for_expert_waves(G, E, pad, W):
    """Host plan arithmetic at the rank counts no CPU process group runs here, and what the expert waves take from it:
    on every owner the sources' rows of an expert are contiguous, disjoint and in rank order inside the expert's padded
    group; every source finds its rows where the owner expects them; the waves' tile ranges (the tile_begin / tile_count
    a wave's GEMM launches get) are whole `pad`-row units and split the owner's tiles without gap or overlap."""
    sys.path[:0] = [os.path.join(ROOT, "test-model-thing-cuda_b200")]
    import tmt_moe_b200 as M
    lib = M.load()
    rng = np.random.default_rng(17 * G + E + W)
    EL = E // G
    W = min(W, EL)
    cnt_all = rng.integers(0, 700, size=(G, E)).astype(np.int32)
    cnt_all[:, rng.integers(0, E)] = 0                      # an expert nobody routes to
    cnt_all[rng.integers(0, G), rng.integers(0, E)] += 5000  # and a hot one
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    plans = []
    for r in range(G):
        tok_poff = np.zeros(E + 1, np.int32); x_counts = np.zeros(EL, np.int32)
        x_poff = np.zeros(EL + 1, np.int32); src_off = np.zeros(G * EL, np.int32)
        rows = lib.tmt_moe_ep_plan(G, r, E, pad, p(cnt_all), p(tok_poff), p(x_counts), p(x_poff), p(src_off))
        assert rows == x_poff[EL]
        plans.append((tok_poff, x_counts, x_poff, src_off.reshape(G, EL)))
    for o, (tok_poff, x_counts, x_poff, src_off) in enumerate(plans):
        assert x_poff[0] == 0 and np.all(x_poff % pad == 0)
        # token side of rank o: its own assignments per expert, padded groups
        np.testing.assert_array_equal(np.diff(tok_poff), (cnt_all[o] + pad - 1) // pad * pad)
        for le in range(EL):
            e = o * EL + le
            assert x_counts[le] == cnt_all[:, e].sum()
            assert x_poff[le + 1] - x_poff[le] == (x_counts[le] + pad - 1) // pad * pad
            # sources in rank order, back to back, from the start of the group
            want = np.concatenate([[0], np.cumsum(cnt_all[:-1, e])])
            np.testing.assert_array_equal(src_off[:, le], want)
        # the waves' GEMM tile ranges on this owner
        covered = 0
        for w in range(W):
            lo, hi = EL * w // W, EL * (w + 1) // W
            assert hi > lo
            begin, count = x_poff[lo] // 128, (x_poff[hi] - x_poff[lo]) // 128
            assert begin == covered and begin % (pad // 128) == 0 and count % (pad // 128) == 0
            covered += count
        assert covered == x_poff[EL] // 128
    # every rank's view of the same thing: capacity verdicts agree with the plans
    worst = max(int(pl[2][EL]) for pl in plans)
    rows_out = ctypes.c_longlong(0)
    assert lib.tmt_moe_ep_check_capacity(G, E, pad, p(cnt_all), ctypes.c_longlong(worst), ctypes.byref(rows_out)) == -1
    bad = lib.tmt_moe_ep_check_capacity(G, E, pad, p(cnt_all), ctypes.c_longlong(worst - pad), ctypes.byref(rows_out))
    assert bad == min(r for r, pl in enumerate(plans) if pl[2][EL] > worst - pad) and rows_out.value == plans[bad][2][EL]


@pytest.mark.parametrize("G,E,K,pad,W,F", [(8, 64, 4, 256, 4, 4), (8, 64, 4, 256, 4, 2), (4, 64, 4, 256, 4, 0), (2, 8, 2, 128, 2, 2)])
def test_peer_addressing_in_expert_waves(G, E, K, pad, W, F):
    """The peer transport's addressing, restated with numpy for rank counts no GPU test here runs: a token-side slot of
    rank r and expert e lives in the owner's buffer at row dest_row0_r[e] + slot - poff_r[e] (group_row in
    csrc/permute.cu), dest_row0 taken from the OWNER's plan; an assignment moves in the wave its expert's index inside
    the owner falls into (in_wave). Sent wave by wave from all ranks, every data row of every owner is written exactly
    once, each expert group holds its sources' rows in rank order and slot order, and what comes back (F waves fetched
    into the token-side copy, the others read by the final combine) is each assignment's own row."""
    sys.path[:0] = [ROOT, os.path.join(ROOT, "test-model-thing-cuda_b200")]
    import tmt_moe_b200 as M
    from oracle import oracle as O
    lib = M.load()
    rng = np.random.default_rng(5 * G + E + W + F)
    EL, T = E // G, 160
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    idx = [np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32) for _ in range(G)]
    lay = [dict(zip(("counts", "off", "poff", "slot_of"), O.layout(i, E, pad))) for i in idx]    # every rank's token side
    cnt_all = np.stack([l["counts"] for l in lay]).astype(np.int32)
    plans = []
    for o in range(G):
        tok_poff = np.zeros(E + 1, np.int32); x_counts = np.zeros(EL, np.int32)
        x_poff = np.zeros(EL + 1, np.int32); src_off = np.zeros(G * EL, np.int32)
        rows = lib.tmt_moe_ep_plan(G, o, E, pad, p(cnt_all), p(tok_poff), p(x_counts), p(x_poff), p(src_off))
        plans.append((int(rows), x_counts, x_poff, src_off.reshape(G, EL)))
        np.testing.assert_array_equal(tok_poff, lay[o]["poff"])
    dest_row0 = [np.array([plans[e // EL][2][e % EL] + plans[e // EL][3][r, e % EL] for e in range(E)]) for r in range(G)]
    ident = lambda r, t: r * 100000 + t + 1                    # a row's content: who sent it
    Xg = [np.zeros(pl[0], np.int64) for pl in plans]
    waves_of = lambda e: [w for w in range(W) if EL * w // W <= e % EL < EL * (w + 1) // W]
    for w in range(W):                                         # dispatch, wave after wave
        for r in range(G):
            for t in range(T):
                for j in range(K):
                    e = int(idx[r][t, j])
                    if waves_of(e) != [w]:
                        continue
                    row = dest_row0[r][e] + lay[r]["slot_of"][t, j] - lay[r]["poff"][e]
                    assert 0 <= row < plans[e // EL][0] and Xg[e // EL][row] == 0
                    Xg[e // EL][row] = ident(r, t)
    for o, (rows, x_counts, x_poff, src_off) in enumerate(plans):
        assert np.count_nonzero(Xg[o]) == x_counts.sum()
        for le in range(EL):
            e = o * EL + le
            want = []
            for s in range(G):                                 # sources in rank order, each in its own slot order
                tj = np.argwhere(idx[s] == e)
                tj = tj[np.argsort(lay[s]["slot_of"][tj[:, 0], tj[:, 1]])]
                want += [ident(s, int(t)) for t, _ in tj]
            np.testing.assert_array_equal(Xg[o][x_poff[le]:x_poff[le] + x_counts[le]], np.array(want, np.int64))
            assert not Xg[o][x_poff[le] + x_counts[le]:x_poff[le + 1]].any()        # pad rows untouched
    Yg = [x * 3 for x in Xg]                                   # the experts' outputs, row for row
    fetched_hi = EL * F // W
    for r in range(G):
        Yr = np.zeros(int(lay[r]["poff"][E]), np.int64)
        for w in range(F):                                     # fetched on the second stream
            for t in range(T):
                for j in range(K):
                    e = int(idx[r][t, j])
                    if waves_of(e) == [w]:
                        slot = lay[r]["slot_of"][t, j]
                        Yr[slot] = Yg[e // EL][dest_row0[r][e] + slot - lay[r]["poff"][e]]
        for t in range(T):                                     # final combine: fetched rows locally, the others from their owners
            for j in range(K):
                e = int(idx[r][t, j])
                slot = lay[r]["slot_of"][t, j]
                got = Yr[slot] if e % EL < fetched_hi else Yg[e // EL][dest_row0[r][e] + slot - lay[r]["poff"][e]]
                assert got == 3 * ident(r, t)


@pytest.mark.parametrize("K", [1, 2, 3, 4, 5, 6, 7, 8])
def test_wave_row_kernel_visits_every_assignment_once(K):
    """The index arithmetic of wave_rows_kernel (csrc/permute.cu) restated: a warp takes 32 / K tokens at a time, lane l
    looks at assignment l of the chunk; for every top-k (also those that do not divide 32) and token counts that do not
    fill the last chunk, each assignment of each token is looked at exactly once, by the lane that the row loop later
    names, and the s_j index of lane j is that assignment's."""
    for T in (1, 31, 32, 33, 257):
        per = 32 // K
        nchunk = (T + per - 1) // per
        blocks, warps = 3, 8
        nwarp = blocks * warps
        seen = np.zeros(T * K, np.int32)
        for gw in range(nwarp):                               # blockIdx.x * warps + warp
            for c in range(gw, nchunk, nwarp):
                for lane in range(32):
                    tl = lane // K
                    t = c * per + tl
                    if tl < per and t < T:
                        a = c * per * K + lane
                        assert a == t * K + lane % K
                        seen[a] += 1
                        # the row loop names this assignment by its lane j: token c * per + j / K, s_j index c * per * K + j
                        assert c * per + lane // K == t and c * per * K + lane == a
        assert (seen == 1).all()
