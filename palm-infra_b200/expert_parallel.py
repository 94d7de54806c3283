"""Expert-parallel routed MoE: one process per GPU, experts split in contiguous blocks.

The reference runs one process on one device (kernels/moe.cpp:576-1129); this is the same op
cut where the experts' outputs meet.  Hidden states and the fp16 router weight are replicated,
so every rank derives the same routes with no dispatch exchange.  Rank r computes the routes
whose expert lies in [r*E/P, (r+1)*E/P) and writes their down-projection outputs into a
[tokens*top_k, H] buffer that is zero everywhere else; one all-reduce (sum) completes the
buffer on every rank -- each row has exactly one owner, so the sum adds only zeros and changes
no bit -- and the ordered combine (fma in ascending expert id, kernels/moe.cpp:1100-1110) then
gives the single-device result bit for bit.

The exchange moves tokens*top_k*H fp32 per layer: 64 KiB for a Qwen3-30B decode token, 16 MiB
for a 256-token prefill.
"""
import numpy as np

from .shard import BLOCK_BYTES, expert_range


def shard_expert_blocks(blocks, num_experts, rows_per_expert, k, rank, world):
    """blocks: flat uint8 BG128 array of an expert aggregate [E*rows_per_expert, K] (expert e
    owns rows e*rows_per_expert..., kernels/moe.cpp:1022-1027) -> (rank's blocks, first
    expert, expert count).  Experts are whole multiples of 8 rows, so the rank's experts are
    one contiguous byte range."""
    if rows_per_expert % 8:
        raise ValueError(f"rows per expert ({rows_per_expert}) must be a multiple of 8")
    lo, hi = expert_range(num_experts, rank, world)
    expert_bytes = (rows_per_expert // 8) * (k // 128) * BLOCK_BYTES
    return blocks[lo * expert_bytes:hi * expert_bytes], lo, hi - lo


class DeviceEngine:
    """The two halves of the op on this rank's GPU, through the C ABI
    (b2w4_moe_expert_outputs / b2w4_moe_combine)."""

    def __init__(self, ctx, router_fp16, gate_up_local, down_local, top_k, intermediate,
                 expert_begin, expert_count):
        self.ctx, self.router = ctx, router_fp16
        self.gate_up, self.down = gate_up_local, down_local
        self.top_k, self.intermediate = top_k, intermediate
        self.expert_begin, self.expert_count = expert_begin, expert_count
        self._buf = {}

    def _buffers(self, hidden):
        import torch
        t, h = hidden.shape
        if t not in self._buf:
            self._buf[t] = (
                torch.empty((t * self.top_k, h), dtype=torch.float32, device=hidden.device),
                torch.empty((t, self.top_k), dtype=torch.int32, device=hidden.device),
                torch.empty((t, self.top_k), dtype=torch.float32, device=hidden.device))
        return self._buf[t]

    def expert_outputs(self, hidden):
        route_out, idx, wts = self._buffers(hidden)
        self.ctx.moe_expert_outputs(hidden, self.router, self.top_k, self.intermediate,
                                    self.gate_up, self.down, self.expert_begin,
                                    self.expert_count, route_out, idx, wts)
        return route_out, idx, wts

    def combine(self, route_out, idx, wts, out):
        self.ctx.moe_combine(route_out, self.top_k, idx, wts, out)


class ExpertParallelMoE:
    """forward(hidden, out): expert outputs on this rank -> all-reduce -> ordered combine.

    `engine` supplies the two compute halves (DeviceEngine on a GPU); `all_reduce` is the
    collective on the route buffer (torch.distributed.all_reduce of the process group, issued
    on the stream the engine's context runs on so the three steps stay stream-ordered)."""

    def __init__(self, engine, all_reduce):
        self.engine = engine
        self.all_reduce = all_reduce

    def forward(self, hidden, out):
        route_out, idx, wts = self.engine.expert_outputs(hidden)
        self.all_reduce(route_out)
        self.engine.combine(route_out, idx, wts, out)
        return out


def build_device_moe(ctx, router_fp16, gate_up_blocks, down_blocks, num_experts, top_k,
                     hidden_size, intermediate, rank, world, all_reduce):
    """Shard the two expert aggregates for `rank`, upload them and return the op."""
    gu, lo, cnt = shard_expert_blocks(gate_up_blocks, num_experts, 2 * intermediate,
                                      hidden_size, rank, world)
    dn, _, _ = shard_expert_blocks(down_blocks, num_experts, hidden_size, intermediate,
                                   rank, world)
    gate_up = ctx.upload_weight(np.ascontiguousarray(gu), cnt * 2 * intermediate, hidden_size)
    down = ctx.upload_weight(np.ascontiguousarray(dn), cnt * hidden_size, intermediate)
    engine = DeviceEngine(ctx, router_fp16, gate_up, down, top_k, intermediate, lo, cnt)
    return ExpertParallelMoE(engine, all_reduce)


class PeerExchangeMoE:
    """forward(hidden, out) with the hand-over inside the kernels (b2w4_moe_forward_ep): the
    owner of a route stores its row, each value tagged with the exchange number, into every
    rank's staging buffer over peer mappings and the combine reads the rows there -- no
    collective call.  Moves 8 bytes per value to every peer, so it is the decode-step variant;
    `stage_rows` (>= tokens*top_k of the largest step) fixes the staging layout for the life
    of the group.  Same bits as ExpertParallelMoE and the single-device op."""

    def __init__(self, engine, group, stage_rows):
        self.engine, self.group, self.stage_rows = engine, group, stage_rows

    @staticmethod
    def stage_words(stage_rows, hidden_size):
        """uint64 words a rank's staging buffer needs (zeroed, 16-byte aligned)."""
        return 2 + 2 * stage_rows * hidden_size

    def forward(self, hidden, out):
        e = self.engine
        if hidden.shape[0] * e.top_k > self.stage_rows:
            raise ValueError("more routes than staging rows")
        e.ctx.moe_forward_ep(hidden, e.router, e.top_k, e.intermediate, e.gate_up, e.down,
                             e.expert_begin, e.expert_count, self.group, self.stage_rows, out)
        return out


class AllToAllMoE:
    """The routed MoE with SEQUENCE-sharded activations: rank r holds its own tokens only
    (contiguous blocks of the sequence, rank order = token order), routes them itself (the
    router is replicated), sends every routed row to the rank that owns its expert, gets the
    expert outputs back the same way and combines its tokens' routes.  Two all-to-all
    exchanges of tokens * top_k rows per layer instead of an all-reduce of the whole route
    buffer; no rank ever holds another rank's hidden states.

    An expert's owner sees all of that expert's rows of the step, in global token order (rows
    arrive by source rank, a rank's rows in its own token order), so the reference's
    per-expert activation rule (per 32 values once an expert holds several rows,
    kernels/moe.cpp:1055-1058) sees the same counts and the result is the one-device result
    bit for bit.

    `engine` supplies three pieces: routes(hidden) -> (indices [T, k], weights [T, k]);
    expert_rows(rows [R, H], experts [R]) -> outputs [R, H] of the local experts (ids relative
    to the rank's first expert, rows of one expert in the order given); combine(route_out
    [T * k, H], indices, weights, out).  The CPU tests supply them from the oracle.  On the
    device, routes and combine exist (b2w4_moe_select_routes after a router matmul,
    b2w4_moe_combine); expert_rows -- the grouped expert matmuls over an explicit row list --
    is inside libb200w4 but not exported yet, so this class is host logic verified on CPU
    ranks only."""

    def __init__(self, engine, dist, rank, world, num_experts, group=None):
        self.engine, self.dist, self.rank, self.world = engine, dist, rank, world
        self.num_experts, self.group = num_experts, group
        if num_experts % world:
            raise ValueError(f"{num_experts} experts do not split over {world} ranks")
        self.per_rank = num_experts // world

    def forward(self, hidden, out):
        import torch
        dist, world, per = self.dist, self.world, self.per_rank
        idx, wts = self.engine.routes(hidden)
        tokens, top_k = idx.shape
        h = hidden.shape[1]
        flat = idx.reshape(-1).to(torch.int64)                 # route (t, j) -> expert
        owner = flat // per
        order = torch.argsort(owner, stable=True)              # by owner, token order inside
        send_counts = torch.bincount(owner, minlength=world)
        recv_counts = torch.zeros_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        send_rows = hidden[order // top_k].contiguous()
        send_experts = (flat[order] - owner[order] * per).contiguous()
        n_recv = int(recv_counts.sum())
        recv_rows = torch.zeros((n_recv, h), dtype=hidden.dtype, device=hidden.device)
        recv_experts = torch.zeros((n_recv,), dtype=torch.int64, device=hidden.device)
        ins, outs = send_counts.tolist(), recv_counts.tolist()
        dist.all_to_all_single(recv_rows, send_rows, output_split_sizes=outs,
                               input_split_sizes=ins, group=self.group)
        dist.all_to_all_single(recv_experts, send_experts, output_split_sizes=outs,
                               input_split_sizes=ins, group=self.group)
        done = self.engine.expert_rows(recv_rows, recv_experts)
        back = torch.zeros_like(send_rows)
        dist.all_to_all_single(back, done.contiguous(), output_split_sizes=ins,
                               input_split_sizes=outs, group=self.group)
        route_out = torch.zeros((tokens * top_k, h), dtype=hidden.dtype, device=hidden.device)
        route_out[order] = back
        self.engine.combine(route_out, idx, wts, out)
        return out
