"""The dense decode step's projection sequence (Qwen3-8B shape by default).

Op order and variants follow decodeStep of the reference
(src/compute/forward.zig:4530-4564 Q/K/V, 5511 O with acc_mode 1,
7377-7390 fused gate+up+SwiGLU, 7420 down with acc_mode 1, 7714 LM head):
seven weight matrices per layer plus the LM head, all batch-1 DMMVs. Attention,
norms and RoPE are not part of this path; their outputs are stood in for by
N(0,1) activation vectors, as the benchmark configuration states.

Tensor parallelism over `world` ranks (one process per GPU): Q/K/V, gate/up
and the LM head are sharded by output rows; O and down are sharded along K
(their input is the local head / FFN slice), so each layer needs two
all-reduces of the hidden vector and the LM head one all-gather. The
collectives are supplied by the caller (`allreduce`, `allgather` callables) so
that this module has no dependency on a communication backend.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional

from . import synth
from ._lib import Q4_K, Q6_K
from .dispatch import Context, DmmvDispatch, row_bytes


@dataclass
class StepShape:
    hidden: int = 4096
    n_layers: int = 36
    q_dim: int = 4096       # 32 heads x 128
    kv_dim: int = 1024      # 8 heads x 128
    ffn: int = 12288
    vocab: int = 151936
    t_attn: int = Q4_K      # Q, K, V, O
    t_gate_up: int = Q4_K
    t_down: int = Q6_K
    t_head: int = Q6_K

    def layer_weight_bytes(self) -> int:
        h = self.hidden
        return ((self.q_dim + 2 * self.kv_dim) * row_bytes(self.t_attn, h) + h * row_bytes(self.t_attn, self.q_dim)
                + 2 * self.ffn * row_bytes(self.t_gate_up, h) + h * row_bytes(self.t_down, self.ffn))

    def weight_bytes(self) -> int:
        """Quantized weight bytes one token reads: the metric's numerator."""
        return self.n_layers * self.layer_weight_bytes() + self.vocab * row_bytes(self.t_head, self.hidden)


QWEN3_8B = StepShape()


@dataclass
class LayerWeights:
    wq: object
    wk: object
    wv: object
    wo: object
    wgate: object
    wup: object
    wdown: object


@dataclass
class DecodeStep:
    """Weights (device tensors), activation buffers and the recorded op sequence of one rank."""
    shape: StepShape
    dd: DmmvDispatch
    rank: int = 0
    world: int = 1
    layers: List[LayerWeights] = field(default_factory=list)
    head: object = None
    # activation buffers (torch tensors)
    x_norm: object = None
    attn_out: object = None
    ffn_act_in: object = None
    q: object = None
    k: object = None
    v: object = None
    act: object = None
    hidden: object = None
    logits: object = None
    allreduce: Optional[Callable] = None   # None with world > 1: the exchange fused into the matvecs (zc_dmmv_push)
    allgather: Optional[Callable] = None

    @staticmethod
    def build(torch, dd: DmmvDispatch, shape: StepShape = QWEN3_8B, rank: int = 0, world: int = 1, seed: int = 2,
              allreduce=None, allgather=None) -> "DecodeStep":
        s, g = shape, world
        for dim, what in ((s.q_dim, "q_dim"), (s.kv_dim, "kv_dim"), (s.ffn, "ffn"), (s.vocab, "vocab")):
            if dim % g:
                raise ValueError(f"{what}={dim} does not divide over {g} ranks")
        if (s.q_dim // g) % 256 or (s.ffn // g) % 256:
            raise ValueError("K shards of O / down must stay multiples of the 256-element super-block")
        dev = f"cuda:{torch.cuda.current_device()}"
        st = DecodeStep(shape=s, dd=dd, rank=rank, world=g, allreduce=allreduce, allgather=allgather)
        base = seed * 100003

        # Every rank generates the same full tensor (the seed does not depend on the rank: the "file" all
        # ranks read) and keeps its shard, cut by the rules of zinc_b200.shard: rows are a contiguous byte
        # range, a K shard is re-laid out as its own dense [M][K / world] tensor.
        def rows(t, M, K, sd):
            w = synth.torch_quant_matrix(t, M, K, dev, sd)
            if g == 1:
                return w
            n = M // g
            return w.view(M, -1)[rank * n:(rank + 1) * n].contiguous().view(-1)

        def kcut(t, M, K, sd):
            w = synth.torch_quant_matrix(t, M, K, dev, sd)
            if g == 1:
                return w
            bs, bpb = synth.BLOCK[t]
            nb = K // bs // g
            return w.view(M, K // bs, bpb)[:, rank * nb:(rank + 1) * nb, :].contiguous().view(-1)

        for layer in range(s.n_layers):
            sd = base + layer * 16
            st.layers.append(LayerWeights(
                wq=rows(s.t_attn, s.q_dim, s.hidden, sd + 0),
                wk=rows(s.t_attn, s.kv_dim, s.hidden, sd + 1),
                wv=rows(s.t_attn, s.kv_dim, s.hidden, sd + 2),
                wo=kcut(s.t_attn, s.hidden, s.q_dim, sd + 3),
                wgate=rows(s.t_gate_up, s.ffn, s.hidden, sd + 4),
                wup=rows(s.t_gate_up, s.ffn, s.hidden, sd + 5),
                wdown=kcut(s.t_down, s.hidden, s.ffn, sd + 6)))
        st.head = rows(s.t_head, s.vocab, s.hidden, base + 99991)
        if g > 1:
            torch.cuda.empty_cache()
        f32 = dict(dtype=torch.float32, device=dev)
        st.x_norm = torch.zeros(s.hidden, **f32)
        st.attn_out = torch.zeros(s.q_dim // g, **f32)
        st.ffn_act_in = torch.zeros(s.ffn // g, **f32)
        st.q = torch.zeros(s.q_dim // g, **f32)
        st.k = torch.zeros(s.kv_dim // g, **f32)
        st.v = torch.zeros(s.kv_dim // g, **f32)
        st.act = torch.zeros(s.ffn // g, **f32)
        st.hidden = torch.zeros(s.hidden, **f32)
        st.logits = torch.zeros(s.vocab, **f32)
        return st

    def local_weight_bytes(self) -> int:
        n = self.head.numel()
        for lw in self.layers:
            n += sum(t.numel() for t in (lw.wq, lw.wk, lw.wv, lw.wo, lw.wgate, lw.wup, lw.wdown))
        return n

    def input_floats(self) -> int:
        return self.x_norm.numel() + self.attn_out.numel() + self.ffn_act_in.numel()

    def record(self) -> int:
        """Enqueue (or, between begin_record/end_record, capture) one token's projections.

        Returns the number of kernels launched by this library."""
        s, dd, g = self.shape, self.dd, self.world
        n0 = dd.ctx.launch_count
        for lw in self.layers:
            # Q, K and V read the same normalised hidden state: one grouped call
            dd.recordDispatchMulti(s.t_attn, [lw.wq, lw.wk, lw.wv], self.x_norm, [self.q, self.k, self.v],
                                   [s.q_dim // g, s.kv_dim // g, s.kv_dim // g], s.hidden)
            if g == 1:
                dd.recordDispatch(s.t_attn, lw.wo, self.attn_out, self.hidden, s.hidden, s.q_dim, acc_mode=1)
            elif self.allreduce is None:  # K-sharded, rows pushed to every rank, summed by the next launch
                dd.recordDispatchPush(s.t_attn, lw.wo, self.attn_out, self.hidden, s.hidden, s.q_dim // g, acc_mode=1)
            else:  # K-sharded: partial sums, then all-reduce into the replicated hidden vector
                # rank 0 adds to the residual, the others overwrite it: the residual enters the sum once
                dd.recordDispatch(s.t_attn, lw.wo, self.attn_out, self.hidden, s.hidden, s.q_dim // g,
                                  acc_mode=1 if self.rank == 0 else 0)
                self.allreduce(self.hidden)
            dd.dispatchDmmvFusedGateUpSwiglu(s.t_gate_up, lw.wgate, lw.wup, self.x_norm, self.act, s.ffn // g,
                                             s.hidden)
            if g == 1:
                dd.recordDispatch(s.t_down, lw.wdown, self.ffn_act_in, self.hidden, s.hidden, s.ffn, acc_mode=1)
            elif self.allreduce is None:
                dd.recordDispatchPush(s.t_down, lw.wdown, self.ffn_act_in, self.hidden, s.hidden, s.ffn // g, acc_mode=1)
            else:
                dd.recordDispatch(s.t_down, lw.wdown, self.ffn_act_in, self.hidden, s.hidden, s.ffn // g,
                                  acc_mode=1 if self.rank == 0 else 0)
                self.allreduce(self.hidden)
        if g == 1:
            dd.recordDispatch(s.t_head, self.head, self.x_norm, self.logits, s.vocab, s.hidden)
        else:
            n = s.vocab // g
            dd.recordDispatch(s.t_head, self.head, self.x_norm, self.logits, n, s.hidden, y_offset=self.rank * n * 4)
            self.allgather(self.logits, self.rank, n)
        return dd.ctx.launch_count - n0
