"""MoE decode layers of the two MoE benchmark configurations, as op sequences over the dispatch mirror.

`QwenMoeLayer`: hidden 2048, 256 routed experts + 1 shared, top-8, expert FFN 512, gate/up Q4_K and
down Q6_K, GPU-side routing with softmax over all experts then renormalisation. Op order follows the
reference's GPU-routed MoE layer (src/compute/forward.zig:6139-6545): router DMMV, softmax_topk,
fused gate+up expert DMMV, SwiGLU, fused down + weighted accumulate, then the shared expert.

`GptOssMoeLayer`: hidden 2880, 32 experts top-4, expert FFN 2880, MXFP4 gate / up / down, router bias
added to the logits, routing by top-k then softmax, per-expert gate / up biases before `swiglu_oai` and a
per-expert down bias inside the weighted sum (src/compute/forward.zig:6712-6930: bias on the router logits
6752-6754, `ffn_gate_exps_bias` / `ffn_up_exps_bias` 6841-6849, `ffn_down_exps_bias` 6923-6927). The
reference walks the selected experts one by one; here every step handles all selected slots in one launch.

Attention, norms and the residual stream are stood in for by fixed N(0,1) vectors, as in the dense
decode step.

Tensor parallelism (world > 1, parallel="tp"): every expert's FFN dimension is cut into per-rank slices on
block boundaries of the down projection's type (`ffn_split`): a rank holds rows [lo, hi) of every expert's
gate and up matrices and the matching K slice of every expert's down matrix, computes a partial hidden
vector per layer, and the ranks sum it (one all-reduce of the hidden vector per layer). The router is
replicated.

Expert parallelism (world > 1, parallel="ep"): rank r holds the whole experts [r E / N, (r+1) E / N). The router
and the top-k run on every rank; `zc_moe_ep_filter` renumbers the selected ids that fall into the rank's range
and marks the other slots "no expert here", which every MoE kernel skips (no weight bytes read, zeros
contributed). The shared expert runs on rank 0. The partial hidden vectors are summed as above.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

from . import synth
from ._lib import F32, MXFP4, Q4_K, Q6_K, ROUTE_SOFTMAX_ALL_RENORM, ROUTE_TOPK_THEN_SOFTMAX
from .dispatch import DmmvDispatch, row_bytes


@dataclass
class MoeShape:
    hidden: int
    n_experts: int
    top_k: int
    ffn: int
    t_gate_up: int
    t_down: int
    rule: int
    shared: bool
    oai: bool
    n_layers: int
    biases: bool = False   # router bias + per-expert gate / up / down biases (GPT-OSS)

    def expert_bytes(self) -> int:
        return 2 * self.ffn * row_bytes(self.t_gate_up, self.hidden) + self.hidden * row_bytes(self.t_down, self.ffn)

    def layer_weight_bytes(self) -> int:
        """Weight bytes one token reads in one layer: selected experts, shared expert, f32 router."""
        return (self.top_k + (1 if self.shared else 0)) * self.expert_bytes() + self.n_experts * self.hidden * 4

    def weight_bytes(self) -> int:
        return self.n_layers * self.layer_weight_bytes()


QWEN35_MOE = MoeShape(hidden=2048, n_experts=256, top_k=8, ffn=512, t_gate_up=Q4_K, t_down=Q6_K,
                      rule=ROUTE_SOFTMAX_ALL_RENORM, shared=True, oai=False, n_layers=40)
GPT_OSS_MOE = MoeShape(hidden=2880, n_experts=32, top_k=4, ffn=2880, t_gate_up=MXFP4, t_down=MXFP4,
                       rule=ROUTE_TOPK_THEN_SOFTMAX, shared=False, oai=True, n_layers=24, biases=True)


def ffn_split(ffn: int, block: int, world: int):
    """Per-rank [lo, hi) element ranges of the FFN dimension: whole blocks of `block` elements, as even as
    the block count allows (the first ranks take the remainder). Raises when a rank would get nothing."""
    if ffn % block:
        raise ValueError("ffn is not a multiple of the block size")
    nb = ffn // block
    if nb < world:
        raise ValueError(f"{nb} blocks of {block} cannot be cut over {world} ranks")
    base, rem = divmod(nb, world)
    out, lo = [], 0
    for r in range(world):
        n = base + (1 if r < rem else 0)
        out.append((lo * block, (lo + n) * block))
        lo += n
    return out


def ep_local_ids(ids, e_lo: int, e_hi: int):
    """Host restatement of the expert-parallel routing filter (`zc_moe_ep_filter`): a numpy array of expert ids
    as the rank that owns [e_lo, e_hi) sees them, renumbered from zero, every other id 0xFFFFFFFF."""
    import numpy as np

    ids = np.asarray(ids, dtype=np.uint32)
    return np.where((ids >= e_lo) & (ids < e_hi), ids - np.uint32(e_lo), np.uint32(0xFFFFFFFF)).astype(np.uint32)


def shard_expert_rows(torch, w, n_experts: int, rows: int, row_nbytes: int, lo: int, hi: int):
    """Rows [lo, hi) of every expert of a stacked [n_experts][rows][row bytes] tensor, stacked again."""
    return w.view(n_experts, rows, row_nbytes)[:, lo:hi, :].contiguous().view(-1)


def shard_expert_k(torch, w, n_experts: int, rows: int, qtype: int, K: int, lo: int, hi: int):
    """Columns [lo, hi) (block aligned) of every row of every expert, re-laid out as dense rows of hi - lo."""
    bs, bpb = synth.BLOCK[qtype]
    return w.view(n_experts * rows, K // bs, bpb)[:, lo // bs:hi // bs, :].contiguous().view(-1)


@dataclass
class MoeLayerWeights:
    router: object
    wg: object
    wu: object
    wd: object
    sg: object = None
    su: object = None
    sd: object = None
    router_bias: object = None   # [n_experts] f32
    bg: object = None            # [n_experts][ffn_local] f32
    bu: object = None
    bd: object = None            # [n_experts][hidden] f32 (rank 0 adds it in a tensor-parallel step)


@dataclass
class MoeDecode:
    shape: MoeShape
    dd: DmmvDispatch
    layers: List[MoeLayerWeights] = field(default_factory=list)
    x: object = None
    hidden: object = None
    logits: object = None
    routing: object = None
    yg: object = None
    yu: object = None
    act: object = None
    sact: object = None
    ffn_local: int = 0
    world: int = 1
    rank: int = 0
    parallel: str = "tp"       # how world > 1 ranks share the experts: "tp" (FFN dimension cut) or "ep" (whole experts)
    allreduce: object = None   # callable(tensor): in-place sum over the ranks
    partial: object = None
    one: object = None
    routing_local: object = None   # expert parallelism: the routing with this rank's experts renumbered, the rest skipped
    e_lo: int = 0
    e_hi: int = 0
    # fused: three launches per layer (router + selection; gate + up + biases + activation with the shared expert as
    # one more slot; down + biases + weighted sum with the shared expert). Off: the reference's dispatch sequence,
    # one launch per dispatch (seven per layer with a shared expert).
    fused: bool = True

    @staticmethod
    def build(torch, dd: DmmvDispatch, shape: MoeShape, seed: int = 3, rank: int = 0, world: int = 1,
              allreduce=None, parallel: str = "tp", fused: bool = True) -> "MoeDecode":
        s = shape
        if parallel not in ("tp", "ep"):
            raise ValueError("parallel must be 'tp' or 'ep'")
        if world == 1:
            parallel = "tp"
        if parallel == "ep" and s.n_experts % world:
            raise ValueError(f"{s.n_experts} experts do not divide over {world} ranks")
        dev = f"cuda:{torch.cuda.current_device()}"
        st = MoeDecode(shape=s, dd=dd, world=world, rank=rank, allreduce=allreduce, parallel=parallel, fused=fused)
        ep = parallel == "ep"
        lo, hi = (0, s.ffn) if ep else ffn_split(s.ffn, synth.BLOCK[s.t_down][0], world)[rank]
        st.e_lo = rank * (s.n_experts // world) if ep else 0
        st.e_hi = (rank + 1) * (s.n_experts // world) if ep else s.n_experts
        st.ffn_local = hi - lo
        rb_h = row_bytes(s.t_gate_up, s.hidden)
        gen = torch.Generator(device=dev).manual_seed(seed)
        for layer in range(s.n_layers):
            sd = seed * 7919 + layer * 16
            w = MoeLayerWeights(
                router=torch.randn(s.n_experts, s.hidden, device=dev, generator=gen) * 0.05,
                wg=synth.torch_quant_matrix(s.t_gate_up, s.n_experts * s.ffn, s.hidden, dev, sd + 0),
                wu=synth.torch_quant_matrix(s.t_gate_up, s.n_experts * s.ffn, s.hidden, dev, sd + 1),
                wd=synth.torch_quant_matrix(s.t_down, s.n_experts * s.hidden, s.ffn, dev, sd + 2))
            if s.shared:
                w.sg = synth.torch_quant_matrix(s.t_gate_up, s.ffn, s.hidden, dev, sd + 3)
                w.su = synth.torch_quant_matrix(s.t_gate_up, s.ffn, s.hidden, dev, sd + 4)
                w.sd = synth.torch_quant_matrix(s.t_down, s.hidden, s.ffn, dev, sd + 5)
            if s.biases:
                w.router_bias = torch.randn(s.n_experts, device=dev, generator=gen) * 0.5
                w.bg = torch.randn(s.n_experts, s.ffn, device=dev, generator=gen)[:, lo:hi].contiguous().view(-1)
                w.bu = torch.randn(s.n_experts, s.ffn, device=dev, generator=gen)[:, lo:hi].contiguous().view(-1)
                w.bd = torch.randn(s.n_experts * s.hidden, device=dev, generator=gen)
            if ep:  # every rank generates the same full tensors and keeps its experts
                eg, ed = s.ffn * rb_h, s.hidden * row_bytes(s.t_down, s.ffn)
                w.wg = w.wg[st.e_lo * eg:st.e_hi * eg].clone()
                w.wu = w.wu[st.e_lo * eg:st.e_hi * eg].clone()
                w.wd = w.wd[st.e_lo * ed:st.e_hi * ed].clone()
                if s.biases:
                    w.bg = w.bg.view(s.n_experts, -1)[st.e_lo:st.e_hi].contiguous().view(-1)
                    w.bu = w.bu.view(s.n_experts, -1)[st.e_lo:st.e_hi].contiguous().view(-1)
                    w.bd = w.bd.view(s.n_experts, -1)[st.e_lo:st.e_hi].contiguous().view(-1)
                if s.shared and rank != 0:
                    w.sg = w.su = w.sd = None
                torch.cuda.empty_cache()
            elif world > 1:  # every rank generates the same full tensors and keeps its slice
                w.wg = shard_expert_rows(torch, w.wg, s.n_experts, s.ffn, rb_h, lo, hi)
                w.wu = shard_expert_rows(torch, w.wu, s.n_experts, s.ffn, rb_h, lo, hi)
                w.wd = shard_expert_k(torch, w.wd, s.n_experts, s.hidden, s.t_down, s.ffn, lo, hi)
                if s.shared:
                    w.sg = shard_expert_rows(torch, w.sg, 1, s.ffn, rb_h, lo, hi)
                    w.su = shard_expert_rows(torch, w.su, 1, s.ffn, rb_h, lo, hi)
                    w.sd = shard_expert_k(torch, w.sd, 1, s.hidden, s.t_down, s.ffn, lo, hi)
                torch.cuda.empty_cache()
            st.layers.append(w)
        f32 = dict(dtype=torch.float32, device=dev)
        st.x = torch.randn(s.hidden, device=dev, generator=gen)
        st.hidden = torch.zeros(s.hidden, **f32)
        st.logits = torch.zeros(s.n_experts, **f32)
        slots = s.top_k + (1 if s.shared and fused else 0)   # fused: the shared expert rides as one more slot
        st.routing = torch.zeros(2 * slots, dtype=torch.int32, device=dev)
        st.routing_local = torch.zeros(2 * slots, dtype=torch.int32, device=dev) if ep else st.routing
        st.yg = torch.zeros(s.top_k * st.ffn_local, **f32)
        st.yu = torch.zeros(s.top_k * st.ffn_local, **f32)
        st.act = torch.zeros(slots * st.ffn_local, **f32)
        st.sact = torch.zeros(st.ffn_local, **f32)
        if world > 1:
            st.partial = torch.zeros(s.hidden, **f32)
            # routing buffer {id 0, weight 1.0} for hidden += partial through moe_weighted_acc
            st.one = torch.tensor([0, 0x3F800000], dtype=torch.int32, device=dev)
        return st

    def record(self) -> int:
        """Enqueue one token's MoE layers; returns the number of kernels launched (collectives included
        when they are the library's own)."""
        s, dd = self.shape, self.dd
        n0 = dd.ctx.launch_count
        f = self.ffn_local
        es_gu = f * row_bytes(s.t_gate_up, s.hidden)
        es_d = s.hidden * row_bytes(s.t_down, f)
        tp = self.world > 1
        ep = self.parallel == "ep" and tp
        n_local = self.e_hi - self.e_lo
        r = self.routing_local
        if self.fused:
            return self._record_fused(es_gu, es_d)
        for w in self.layers:
            dd.recordDispatch(F32, w.router, self.x, self.logits, s.n_experts, s.hidden)
            dd.dispatchSoftmaxTopk(self.logits, self.routing, s.n_experts, s.top_k, rule=s.rule, bias=w.router_bias)
            if ep:
                dd.dispatchMoeEpFilter(self.routing, r, s.top_k, self.e_lo, self.e_hi)
            dd.dispatchMoeFusedGateUp(s.t_gate_up, w.wg, w.wu, self.x, self.yg, self.yu, r, f,
                                      s.hidden, es_gu, s.top_k, 0)
            if s.biases:
                dd.dispatchMoeBiasAct(self.yg, self.yu, w.bg, w.bu, r, self.act, f, s.top_k,
                                      n_local, oai=s.oai)
            else:
                dd.dispatchSwiglu(self.yg, self.yu, self.act, s.top_k * f, oai=s.oai)
            acc = self.partial if tp else self.hidden
            if tp:
                dd.ctx.memset(_as_buffer(self.partial), 0)
            dd.dispatchMoeFusedDownAcc(s.t_down, w.wd, self.act, acc, r, s.hidden, f, es_d, s.top_k, f)
            if s.biases and (ep or self.rank == 0):  # tp: the bias enters once; ep: with the rank's own experts
                dd.dispatchMoeWeightedBiasAcc(acc, w.bd, r, s.hidden, s.top_k, n_local)
            if s.shared and w.sg is not None:
                dd.dispatchDmmvFusedGateUpSwiglu(s.t_gate_up, w.sg, w.su, self.x, self.sact, f, s.hidden)
                dd.recordDispatch(s.t_down, w.sd, self.sact, acc, s.hidden, f, acc_mode=1)
            if tp:
                if self.allreduce is not None:
                    self.allreduce(self.partial)
                dd.dispatchMoeWeightedAcc(self.hidden, self.partial, self.one, s.hidden, 1, s.hidden)
        return dd.ctx.launch_count - n0

    def _record_fused(self, es_gu: int, es_d: int) -> int:
        s, dd, f = self.shape, self.dd, self.ffn_local
        n0 = dd.ctx.launch_count
        tp = self.world > 1
        ep = self.parallel == "ep" and tp
        slots = s.top_k + (1 if s.shared else 0)
        r = self.routing_local
        for w in self.layers:
            acc = self.partial if tp else self.hidden
            if tp:
                dd.ctx.memset(_as_buffer(self.partial), 0)
            # router + selection (+ the rank's view of it under expert parallelism; the shared expert on rank 0)
            dd.dispatchMoeRouterTopk(self.x, w.router, self.logits, self.routing, s.n_experts, s.hidden, s.top_k,
                                     rule=s.rule, bias=w.router_bias, shared_slot=s.shared,
                                     routing_local=r if ep else None, e_lo=self.e_lo, e_hi=self.e_hi,
                                     local_shared=w.sg is not None)
            shared_gu = (w.sg, w.su) if s.shared and w.sg is not None else None
            dd.dispatchMoeGateUpActEx(s.t_gate_up, w.wg, w.wu, self.x, self.act, r, f, s.hidden, es_gu, slots,
                                      shared=shared_gu, biases=(w.bg, w.bu) if s.biases else None, oai=s.oai)
            # tensor parallelism: the down bias enters once (rank 0); expert parallelism: with the rank's own experts
            bias_d = w.bd if s.biases and (ep or not tp or self.rank == 0) else None
            dd.dispatchMoeDownAccEx(s.t_down, w.wd, self.act, acc, r, s.hidden, f, es_d, slots, f,
                                    shared=w.sd if s.shared and w.sg is not None else None, bias=bias_d)
            if tp:
                if self.allreduce is not None:
                    self.allreduce(self.partial)
                dd.dispatchMoeWeightedAcc(self.hidden, self.partial, self.one, s.hidden, 1, s.hidden)
        return dd.ctx.launch_count - n0


@dataclass
class MoePrefill:
    """The routed experts of one MoE layer over a prefill batch of T tokens: gate and up of every (token, slot)
    pair grouped by expert on the tensor cores, activation, down, and the weighted sum of a token's slots back
    into its hidden row (the grouped path of src/shaders/metal/moe_route_pack.metal, dmmv_q4k_moe_cols.metal,
    moe_route_scatter.metal). The routing ids are the selection of N(0,1) logits.

    Expert parallelism (world > 1): tokens and routing are replicated; rank r holds the whole experts
    [r E / N, (r+1) E / N), filters the routing to them (`zc_moe_ep_filter`: local ids, the other slots marked
    absent), runs the same calls on its own stack (pairs of absent slots are neither grouped nor computed, and the
    weighted sum leaves them out), and the ranks' partial [T][hidden] outputs are summed by `allreduce` (a
    bandwidth-bound sum of T * hidden floats: NCCL)."""
    shape: MoeShape
    dd: DmmvDispatch
    T: int
    rank: int = 0
    world: int = 1
    e_lo: int = 0
    e_hi: int = 0
    wg: object = None
    wu: object = None
    wd: object = None
    X: object = None
    routing: object = None        # [T][2k] ids + weights of the global selection
    routing_local: object = None  # the same as this rank sees it
    ids_local: object = None      # [T][k] flattened id table of the cross-token calls
    gate: object = None
    up: object = None
    act: object = None
    down: object = None
    hidden: object = None
    workspace: object = None
    allreduce: object = None

    @staticmethod
    def build(torch, dd: DmmvDispatch, shape: MoeShape, T: int, seed: int = 5, rank: int = 0, world: int = 1,
              allreduce=None, local_only: bool = False) -> "MoePrefill":
        s = shape
        if s.n_experts % world:
            raise ValueError(f"{s.n_experts} experts do not divide over {world} ranks")
        dev = f"cuda:{torch.cuda.current_device()}"
        n_local = s.n_experts // world
        st = MoePrefill(shape=s, dd=dd, T=T, rank=rank, world=world, allreduce=allreduce,
                        e_lo=rank * n_local, e_hi=(rank + 1) * n_local)
        eg = s.ffn * row_bytes(s.t_gate_up, s.hidden)
        ed = s.hidden * row_bytes(s.t_down, s.ffn)
        if local_only and world > 1:   # benchmark: only this rank's experts are ever generated
            st.wg = synth.torch_quant_matrix(s.t_gate_up, n_local * s.ffn, s.hidden, dev, seed * 31 + 3 * rank)
            st.wu = synth.torch_quant_matrix(s.t_gate_up, n_local * s.ffn, s.hidden, dev, seed * 31 + 3 * rank + 1)
            st.wd = synth.torch_quant_matrix(s.t_down, n_local * s.hidden, s.ffn, dev, seed * 31 + 3 * rank + 2)
        else:                           # every rank cuts its experts out of the same seeded full tensors
            wg = synth.torch_quant_matrix(s.t_gate_up, s.n_experts * s.ffn, s.hidden, dev, seed * 31)
            wu = synth.torch_quant_matrix(s.t_gate_up, s.n_experts * s.ffn, s.hidden, dev, seed * 31 + 1)
            wd = synth.torch_quant_matrix(s.t_down, s.n_experts * s.hidden, s.ffn, dev, seed * 31 + 2)
            st.wg = wg[st.e_lo * eg:st.e_hi * eg].clone()
            st.wu = wu[st.e_lo * eg:st.e_hi * eg].clone()
            st.wd = wd[st.e_lo * ed:st.e_hi * ed].clone()
            del wg, wu, wd
            torch.cuda.empty_cache()
        gen = torch.Generator(device=dev).manual_seed(seed)   # the same tokens and routing on every rank
        k = s.top_k
        st.X = torch.randn(T, s.hidden, device=dev, generator=gen)
        logits = torch.randn(T, s.n_experts, device=dev, generator=gen)
        st.routing = torch.zeros(T * 2 * k, dtype=torch.int32, device=dev)
        dd.dispatchSoftmaxTopk(logits, st.routing, s.n_experts, k, s.rule, T)
        if world > 1:
            st.routing_local = torch.zeros(T * 2 * k, dtype=torch.int32, device=dev)
            st.ids_local = torch.zeros(T * k, dtype=torch.int32, device=dev)
        else:
            dd.ctx.submit_and_wait()
            st.routing_local = st.routing
            st.ids_local = st.routing.view(T, 2 * k)[:, :k].contiguous().view(-1)
        f32 = dict(dtype=torch.float32, device=dev)
        st.gate = torch.zeros(T * k * s.ffn, **f32)
        st.up = torch.zeros(T * k * s.ffn, **f32)
        st.act = torch.zeros(T * k * s.ffn, **f32)
        st.down = torch.zeros(T * k * s.hidden, **f32)
        st.hidden = torch.zeros(T * s.hidden, **f32)
        st.workspace = torch.empty(max(dd.moeGroupedWorkspaceBytes(T, k, s.hidden, n_local),
                                       dd.moeGroupedWorkspaceBytes(T * k, 1, s.ffn, n_local)),
                                   dtype=torch.uint8, device=dev)
        return st

    def record(self) -> int:
        """Enqueue the layer (the workspace must be set: `dd.setWorkspace(self.workspace)`); hidden += result.
        Returns the number of the library's kernels launched."""
        s, dd, T, k = self.shape, self.dd, self.T, self.shape.top_k
        n0 = dd.ctx.launch_count
        n_local = self.e_hi - self.e_lo
        eg = s.ffn * row_bytes(s.t_gate_up, s.hidden)
        ed = s.hidden * row_bytes(s.t_down, s.ffn)
        if self.world > 1:
            dd.ctx.memset(_as_buffer(self.hidden), 0)
            dd.dispatchMoeEpFilter(self.routing, self.routing_local, k, self.e_lo, self.e_hi, n_tokens=T)
            dd.dispatchMoeEpFilter(self.routing, self.ids_local, k, self.e_lo, self.e_hi, n_tokens=T, out_stride=k)
        dd.recordMoeBatchedDispatchPair(s.t_gate_up, self.wg, self.wu, self.X, self.gate, self.up, self.ids_local,
                                        s.ffn, s.hidden, eg, n_local, k, T, s.hidden, k * s.ffn)
        dd.dispatchSwiglu(self.gate, self.up, self.act, T * k * s.ffn, oai=s.oai)
        dd.recordMoeBatchedDispatch(s.t_down, self.wd, self.act, self.down, self.ids_local, s.hidden, s.ffn, ed,
                                    n_local, 1, T * k, s.ffn, s.hidden)
        dd.dispatchMoeRouteScatter(self.routing_local, self.down, self.hidden, T, s.hidden, k, 2 * k)
        n = dd.ctx.launch_count - n0
        if self.world > 1 and self.allreduce is not None:
            self.allreduce(self.hidden)
        return n


def _as_buffer(t):
    from .dispatch import Buffer
    return Buffer.from_torch(t)
