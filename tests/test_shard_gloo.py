"""Tensor-parallel host logic on two CPU ranks (gloo): each rank cuts its shard from the same GGUF
tensor with zinc_b200.shard, the oracle stands in for the device matvec, and the collectives the
decode step uses (all-gather for row shards, all-reduce for K shards, the FFN pairing
gate/up row-sharded -> local SwiGLU -> down K-sharded) must reproduce the single-rank result."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import zinc_b200 as zb
    from oracle import oracle as zo
    from zinc_b200 import shard, synth

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        res = {}
        hidden, ffn = 512, 1024
        g = synth.rng(300, 0)  # the same stream on every rank: the "file" all ranks read
        wg = synth.quant_matrix(g, zb.Q4_K, ffn, hidden)
        wu = synth.quant_matrix(g, zb.Q4_K, ffn, hidden)
        wd = synth.quant_matrix(g, zb.Q6_K, hidden, ffn)
        x = synth.activations(g, hidden)
        # single-rank result
        act_full = zo.swiglu(zo.dmmv_f64(wg, zb.Q4_K, ffn, hidden, x).astype(np.float32),
                             zo.dmmv_f64(wu, zb.Q4_K, ffn, hidden, x).astype(np.float32))
        y_full = zo.dmmv_f64(wd, zb.Q6_K, hidden, ffn, act_full)

        # row shard + all-gather
        p = shard.plan("row", ffn, hidden, zb.Q4_K, rank, world)
        gl = zo.dmmv_f64(shard.row_shard(wg, zb.Q4_K, ffn, hidden, rank, world), zb.Q4_K, p.M, p.K, x)
        parts = [torch.zeros(p.M, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(gl))
        res["row_gather"] = float(np.abs(torch.cat(parts).numpy() - zo.dmmv_f64(wg, zb.Q4_K, ffn, hidden, x)).max())

        # FFN pairing: local SwiGLU on the local rows, down K-sharded over the same slice, one all-reduce
        ul = zo.dmmv_f64(shard.row_shard(wu, zb.Q4_K, ffn, hidden, rank, world), zb.Q4_K, p.M, p.K, x)
        act_local = zo.swiglu(gl.astype(np.float32), ul.astype(np.float32))
        pk = shard.plan("k", hidden, ffn, zb.Q6_K, rank, world)
        assert (pk.x_begin, pk.K) == (p.y_begin, p.M)  # the K slice of down is this rank's gate/up row slice
        yl = zo.dmmv_f64(shard.k_shard(wd, zb.Q6_K, hidden, ffn, rank, world), zb.Q6_K, pk.M, pk.K, act_local)
        t = torch.from_numpy(yl.copy())
        dist.all_reduce(t)
        res["ffn_pair"] = float(np.abs(t.numpy() - y_full).max() / np.abs(y_full).max())

        # MoE experts, tensor parallel: every expert's FFN dimension cut on down-projection blocks
        # (uneven: 5 MXFP4 blocks over 2 ranks), partial hidden vectors summed by one all-reduce
        from zinc_b200 import moe_step

        E, H, F, k = 4, 256, 160, 2
        wg_e = synth.quant_matrix(g, zb.MXFP4, E * F, H)
        wu_e = synth.quant_matrix(g, zb.MXFP4, E * F, H)
        wd_e = synth.quant_matrix(g, zb.MXFP4, E * H, F)
        ids = np.array([2, 0], np.uint32)
        wts = np.array([0.7, 0.3], np.float64)
        sg, sdn = zb.expert_slice_bytes(zb.MXFP4, F, H), zb.expert_slice_bytes(zb.MXFP4, H, F)
        xr = np.repeat(x[None, :H], k, axis=0)

        def moe(wg_, wu_, wd_, f):
            s_g, s_d = zb.expert_slice_bytes(zb.MXFP4, f, H), zb.expert_slice_bytes(zb.MXFP4, H, f)
            gate = zo.moe_dmmv_f64(wg_, zb.MXFP4, f, H, s_g, ids, H, xr).astype(np.float32)
            up = zo.moe_dmmv_f64(wu_, zb.MXFP4, f, H, s_g, ids, H, xr).astype(np.float32)
            act = zo.swiglu(gate.reshape(-1), up.reshape(-1)).reshape(k, f)
            return (wts[:, None] * zo.moe_dmmv_f64(wd_, zb.MXFP4, H, f, s_d, ids, f, act)).sum(0)

        full = moe(wg_e, wu_e, wd_e, F)
        cuts = moe_step.ffn_split(F, 32, world)
        assert cuts == [(0, 96), (96, 160)]
        lo, hi = cuts[rank]
        tw = lambda a: torch.from_numpy(a)
        wg_l = moe_step.shard_expert_rows(torch, tw(wg_e), E, F, sg // F, lo, hi).numpy()
        wu_l = moe_step.shard_expert_rows(torch, tw(wu_e), E, F, sg // F, lo, hi).numpy()
        wd_l = moe_step.shard_expert_k(torch, tw(wd_e), E, H, zb.MXFP4, F, lo, hi).numpy()
        tm = torch.from_numpy(moe(wg_l, wu_l, wd_l, hi - lo).copy())
        dist.all_reduce(tm)
        res["moe_tp"] = float(np.abs(tm.numpy() - full).max() / np.abs(full).max())

        # MoE experts, expert parallel: rank r holds the whole experts [r E / N, (r+1) E / N); the routing filter
        # renumbers the selected ids in that range and skips the others; partial hidden vectors are summed
        e_lo, e_hi = rank * E // world, (rank + 1) * E // world
        keep = (ids >= e_lo) & (ids < e_hi)
        if keep.any():
            lids = (ids[keep] - e_lo).astype(np.uint32)
            kk = int(keep.sum())
            xl = np.repeat(x[None, :H], kk, axis=0)
            wg_p, wu_p, wd_p = wg_e[e_lo * sg:e_hi * sg], wu_e[e_lo * sg:e_hi * sg], wd_e[e_lo * sdn:e_hi * sdn]
            gate = zo.moe_dmmv_f64(wg_p, zb.MXFP4, F, H, sg, lids, H, xl).astype(np.float32)
            up = zo.moe_dmmv_f64(wu_p, zb.MXFP4, F, H, sg, lids, H, xl).astype(np.float32)
            act = zo.swiglu(gate.reshape(-1), up.reshape(-1)).reshape(kk, F)
            mine = (wts[keep][:, None] * zo.moe_dmmv_f64(wd_p, zb.MXFP4, H, F, sdn, lids, F, act)).sum(0)
        else:
            mine = np.zeros(H)
        te = torch.from_numpy(np.ascontiguousarray(mine))
        dist.all_reduce(te)
        res["moe_ep"] = float(np.abs(te.numpy() - full).max() / np.abs(full).max())

        # the same over a prefill batch: tokens and routing replicated, a rank computes the pairs of its own experts
        # only, the [T][H] partial outputs are summed
        T = 5
        ids_t = np.stack([g.choice(E, size=k, replace=False) for _ in range(T)]).astype(np.uint32)
        wts_t = g.random((T, k))
        X_t = synth.activations(g, T, H)

        def pair_out(wg_, wu_, wd_, e, xrow):
            one = np.array([e], np.uint32)
            gate = zo.moe_dmmv_f64(wg_, zb.MXFP4, F, H, sg, one, H, xrow[None]).astype(np.float32)
            up = zo.moe_dmmv_f64(wu_, zb.MXFP4, F, H, sg, one, H, xrow[None]).astype(np.float32)
            act = zo.swiglu(gate.reshape(-1), up.reshape(-1)).reshape(1, F)
            return zo.moe_dmmv_f64(wd_, zb.MXFP4, H, F, sdn, one, F, act)[0]

        full_t = np.zeros((T, H))
        for t in range(T):
            for s in range(k):
                full_t[t] += wts_t[t, s] * pair_out(wg_e, wu_e, wd_e, ids_t[t, s], X_t[t])
        local = moe_step.ep_local_ids(ids_t, e_lo, e_hi)
        wg_p, wu_p, wd_p = wg_e[e_lo * sg:e_hi * sg], wu_e[e_lo * sg:e_hi * sg], wd_e[e_lo * sdn:e_hi * sdn]
        mine_t = np.zeros((T, H))
        for t in range(T):
            for s in range(k):
                if local[t, s] != 0xFFFFFFFF:
                    mine_t[t] += wts_t[t, s] * pair_out(wg_p, wu_p, wd_p, local[t, s], X_t[t])
        tp_ = torch.from_numpy(mine_t)
        dist.all_reduce(tp_)
        res["moe_ep_prefill"] = float(np.abs(tp_.numpy() - full_t).max() / np.abs(full_t).max())

        # refusals
        for fn, args in ((shard.row_range, (5, rank, world)), (shard.k_range, (zb.Q6_K, 768, rank, world))):
            try:
                fn(*args)
                res["refusal"] = False
            except ValueError:
                res.setdefault("refusal", True)
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_tensor_parallel_ffn():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = dict(q.get(timeout=150) for _ in procs)
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    for r in range(2):
        assert out[r]["row_gather"] == 0.0
        assert out[r]["ffn_pair"] <= 1e-12
        assert out[r]["moe_tp"] <= 1e-6   # f32 SwiGLU outputs feed the down projection
        assert out[r]["moe_ep"] <= 1e-12  # whole experts: the same numbers, summed in another order
        assert out[r]["moe_ep_prefill"] <= 1e-12
        assert out[r]["refusal"] is True


def test_moe_ffn_split():
    sys.path.insert(0, ROOT)
    from zinc_b200.moe_step import ffn_split

    assert ffn_split(2880, 32, 4) == [(0, 736), (736, 1472), (1472, 2176), (2176, 2880)]  # 23, 23, 22, 22 blocks
    assert ffn_split(512, 256, 2) == [(0, 256), (256, 512)]
    with pytest.raises(ValueError):
        ffn_split(512, 256, 4)   # two Q6_K blocks cannot feed four ranks
    with pytest.raises(ValueError):
        ffn_split(100, 32, 2)


def test_shards_are_byte_ranges():
    sys.path.insert(0, ROOT)
    import zinc_b200 as zb
    from zinc_b200 import shard, synth

    g = synth.rng(301, 0)
    M, K = 12, 1024
    w = synth.quant_matrix(g, zb.Q5_K, M, K)
    rb = zb.row_bytes(zb.Q5_K, K)
    flat = w.reshape(-1)
    for world in (1, 2, 4):
        got = np.concatenate([shard.row_shard(w, zb.Q5_K, M, K, r, world) for r in range(world)])
        assert np.array_equal(got, flat)
        ks = [shard.k_shard(w, zb.Q5_K, M, K, r, world).reshape(M, -1) for r in range(world)]
        assert np.array_equal(np.concatenate(ks, axis=1).reshape(-1), flat)
        assert all(k.shape[1] == rb // world for k in ks)


def test_moe_bytes_per_token():
    """Weight bytes one token reads per MoE layer: routed experts + shared expert + f32 router."""
    sys.path.insert(0, ROOT)
    from zinc_b200.moe_step import GPT_OSS_MOE, QWEN35_MOE

    assert QWEN35_MOE.expert_bytes() == 2_039_808
    assert QWEN35_MOE.layer_weight_bytes() == 8 * 2_039_808 + 2_039_808 + 2_097_152
    assert GPT_OSS_MOE.expert_bytes() == 3 * 4_406_400
    assert GPT_OSS_MOE.layer_weight_bytes() == 52_876_800 + 32 * 2880 * 4
