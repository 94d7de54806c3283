"""A Qwen3-shaped decoder (dense, or with a routed mixture of experts as the feed-forward
block) driven through the C ABI: embedding rows, per layer RMSNorm ->
fused qkv matmul -> per-head Q/K RMSNorm -> rotary embedding -> KV append + causal attention ->
o matmul -> residual add + RMSNorm -> gate_up matmul -> SwiGLU -> down matmul (or the MOE
operator in their place) -> residual add (+ next RMSNorm), final norm, lm_head with the greedy
token picked on the device.  The layer structure is the reference's graph builder's
(models/qwen3.py:171-345; the mixture-of-experts block: models/qwen3_moe.py); every operator is a
libb200w4 kernel, nothing runs on the host between the first embedding row and the token.

This is the host-side mirror of what the reference's engine does per step for benchmark
configuration 3 (engine/engine.cpp prefill / decode), reduced to greedy decoding on synthetic
weights; torch provides device memory only.

Activation rule of the matmuls: the reference's -- per 128 values for one row (decode), per 32
values for several (prefill) -- unless `multi_row_rule` says otherwise.
"""
import numpy as np

from . import capi, synth


class DecoderConfig:
    def __init__(self, layers, hidden, heads, kv_heads, head_dim, intermediate, vocab,
                 rope_theta=1e6, eps=1e-6, experts=0, top_k=0):
        """experts > 0: every layer's feed-forward block is the routed mixture of experts
        (softmax top-k router, `experts` SwiGLU experts of width `intermediate`)."""
        self.layers, self.hidden, self.heads, self.kv_heads = layers, hidden, heads, kv_heads
        self.head_dim, self.intermediate, self.vocab = head_dim, intermediate, vocab
        self.rope_theta, self.eps = rope_theta, eps
        self.experts, self.top_k = experts, top_k
        self.q_dim, self.kv_dim = heads * head_dim, kv_heads * head_dim

    @staticmethod
    def qwen3_4b():
        """Benchmark configuration 3: 36 layers, hidden 2560, 32 q / 8 kv heads of 128,
        SwiGLU intermediate 9728, vocabulary 151936, rope theta 1e6."""
        return DecoderConfig(36, 2560, 32, 8, 128, 9728, 151936)

    @staticmethod
    def qwen3_30b_a3b():
        """Benchmark configuration 4: 48 layers, hidden 2048, 32 q / 4 kv heads of 128, 128
        experts of width 768 with 8 routed per token, vocabulary 151936."""
        return DecoderConfig(48, 2048, 32, 4, 128, 768, 151936, experts=128, top_k=8)

    @staticmethod
    def qwen3_235b_a22b():
        """Benchmark configuration 5: 94 layers, hidden 4096, 64 q / 4 kv heads of 128, 128
        experts of width 1536 with 8 routed per token, vocabulary 151936: 121 GB of W4G128
        weights, which one GPU's 180 GB holds."""
        return DecoderConfig(94, 4096, 64, 4, 128, 1536, 151936, experts=128, top_k=8)


def rope_tables(positions, rope_dim, theta):
    """cos / sin [len(positions), rope_dim // 2] as the reference fills them on the host
    (engine/input_prep.cpp:18-31): theta_i = 1 / theta^(2i / rope_dim), angle = pos * theta_i,
    all in fp32 through the host libm's float functions (b2w4_rope_tables: numpy's float
    cosine and sine differ from a libm's in the last bit for a third of the entries).
    `positions`: consecutive integers."""
    positions = list(positions)
    if positions != list(range(positions[0], positions[0] + len(positions))):
        raise ValueError("positions must be consecutive")
    return capi.rope_tables(len(positions), positions[0], rope_dim, theta)


def synthetic_weights(cfg, seed=20261125, distinct_layers=None, lazy=False):
    """Host-side synthetic model: BG128 blocks for every matmul weight, fp16 embedding rows and
    router rows, fp32 norm weights.  distinct_layers < cfg.layers generates that many layers
    and gives the others the same blocks rotated by whole blocks (a different weight per layer
    at a fraction of the generation time).  lazy: "layers" is a generator, so that a model of
    tens of gigabytes is uploaded layer by layer without ever being whole in host memory."""
    d = distinct_layers or cfg.layers
    # mixture of experts: the aggregates hold expert e's rows at [e * rows, (e + 1) * rows)
    per = max(1, cfg.experts)
    shapes = {"qkv": (cfg.q_dim + 2 * cfg.kv_dim, cfg.hidden), "o": (cfg.hidden, cfg.q_dim),
              "gate_up": (per * 2 * cfg.intermediate, cfg.hidden),
              "down": (per * cfg.hidden, cfg.intermediate)}
    base = {}

    def layer(l):
        if l % d not in base:
            base[l % d] = {k: synth.bg128_weight(seed, 1000 + 10 * (l % d) + j, n, kk)
                           for j, (k, (n, kk)) in enumerate(shapes.items())}
        src = base[l % d]
        w = {k: (v if l < d else np.roll(v, 544 * (l // d))) for k, v in src.items()}
        rng = np.random.default_rng(seed + 7 * l)
        for name, n in (("ln1", cfg.hidden), ("ln2", cfg.hidden), ("q_norm", cfg.head_dim),
                        ("k_norm", cfg.head_dim)):
            w[name] = (1.0 + 0.05 * rng.standard_normal(n)).astype(np.float32)
        if cfg.experts:
            w["router"] = synth.router_weight(seed, 2000 + l, cfg.experts, cfg.hidden)
        return w

    layers = (layer(l) for l in range(cfg.layers))
    rng = np.random.default_rng(seed + 99)
    return {"shapes": shapes, "layers": layers if lazy else list(layers),
            "final_norm": (1.0 + 0.05 * rng.standard_normal(cfg.hidden)).astype(np.float32),
            "embed": _embedding(seed, cfg),
            "lm_head": synth.bg128_weight(seed, 901, cfg.vocab, cfg.hidden)}


def _embedding(seed, cfg, distinct_rows=8192):
    """fp16 N(0, 0.02) rows [vocab, hidden]; beyond `distinct_rows` the rows repeat, rotated by
    one element per repetition."""
    rows = min(cfg.vocab, distinct_rows)
    base = synth.router_weight(seed, 900, rows, cfg.hidden)
    if rows == cfg.vocab:
        return base
    parts = [np.roll(base, rep, axis=1) for rep in range((cfg.vocab + rows - 1) // rows)]
    return np.ascontiguousarray(np.concatenate(parts)[:cfg.vocab])


class DenseDecoder:
    def __init__(self, ctx, cfg, weights, capacity, multi_row_rule=capi.ACT_G32, fused_qkv=None,
                 device="cuda"):
        """device: where torch keeps the tensors the operators work on ("cuda" with the C ABI
        context; the multi-rank tests run the same driver on "cpu" with a context made of the
        CPU oracle)."""
        import torch
        self.torch, self.ctx, self.cfg, self.capacity = torch, ctx, cfg, capacity
        self.device = device
        self.multi_row_rule = multi_row_rule
        can_fuse = cfg.head_dim % 64 == 0 and cfg.head_dim <= 256
        self.fused_qkv = can_fuse if fused_qkv is None else (fused_qkv and can_fuse)
        sh = weights["shapes"]
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
        self.layers = []
        for w in weights["layers"]:
            self.layers.append({
                **{k: ctx.upload_weight(w[k], *sh[k]) for k in sh},
                **{k: dev(w[k]) for k in ("ln1", "ln2", "q_norm", "k_norm")},
                **({"router": dev(w["router"].view(np.int16))} if cfg.experts else {}),
                "k_cache": torch.zeros((cfg.kv_heads, capacity, cfg.head_dim), device=device),
                "v_cache": torch.zeros((cfg.kv_heads, capacity, cfg.head_dim), device=device)})
        self.final_norm = dev(weights["final_norm"])
        self.embed = dev(weights["embed"].view(np.int16))
        self.lm_head = ctx.upload_weight(weights["lm_head"], cfg.vocab, cfg.hidden)
        cos, sin = rope_tables(range(capacity), cfg.head_dim, cfg.rope_theta)
        self.cos, self.sin = dev(cos), dev(sin)  # rows = positions
        self.past = 0
        self.token = torch.zeros((1,), dtype=torch.int32, device=device)
        self.past_dev = torch.zeros((1,), dtype=torch.int32, device=device)
        self.history = torch.zeros((capacity,), dtype=torch.int32, device=device)
        self.step_graph = None
        self._buf = {}

    def _b(self, name, rows, cols):
        key = (name, rows, cols)
        if key not in self._buf:
            self._buf[key] = self.torch.empty((rows, cols), dtype=self.torch.float32,
                                              device=self.device)
        return self._buf[key]

    def reset(self):
        self.past = 0

    def forward(self, ids_dev, tokens, on_device_position=False):
        """Runs `tokens` new tokens (int32 ids on the device) through the decoder and leaves
        the greedy next token in self.token.  Asynchronous.  on_device_position: the position
        comes from self.past_dev inside the kernels (the form a CUDA graph can replay)."""
        c, cfg, ctx = self.ctx, self.cfg, self.ctx
        T, H, D = tokens, cfg.hidden, cfg.head_dim
        rule = capi.ACT_G128 if T == 1 else self.multi_row_rule
        pos_dev = self.past_dev if on_device_position else None
        x = self._b("x", T, H)
        h = self._b("h", T, H)
        qkv = self._b("qkv", T, cfg.q_dim + 2 * cfg.kv_dim)
        q, k, v = self._b("q", T, cfg.q_dim), self._b("k", T, cfg.kv_dim), self._b("v", T, cfg.kv_dim)
        attn, o = self._b("attn", T, cfg.q_dim), self._b("o", T, H)
        gu = act = None
        if not cfg.experts:
            gu, act = self._b("gu", T, 2 * cfg.intermediate), self._b("act", T, cfg.intermediate)
        dn = self._b("dn", T, H)
        c.embed_rows(self.embed, ids_dev, x)
        c.rms_norm(x, self.layers[0]["ln1"], cfg.eps, h)
        for li, L in enumerate(self.layers):
            c.matmul(L["qkv"], h, qkv, rule=rule)
            if self.fused_qkv:  # norm + rotary embedding + cache append in one launch
                c.qkv_prepare(qkv, T, cfg.heads, cfg.kv_heads, D, L["q_norm"], L["k_norm"],
                              cfg.eps, self.cos, self.sin, self.past, q, L["k_cache"],
                              L["v_cache"], self.capacity, pos_dev)
                c.attention(q, None, None, L["k_cache"], L["v_cache"], attn, T, cfg.heads,
                            cfg.kv_heads, D, self.past, self.capacity, D ** -0.5, pos_dev)
            else:           # the same step operator by operator
                c.copy_rows(qkv, q, T, cfg.q_dim)
                c.copy_rows(qkv[:, cfg.q_dim:], k, T, cfg.kv_dim)
                c.copy_rows(qkv[:, cfg.q_dim + cfg.kv_dim:], v, T, cfg.kv_dim)
                qh, kh = q.view(T * cfg.heads, D), k.view(T * cfg.kv_heads, D)
                c.rms_norm(qh, L["q_norm"], cfg.eps, qh)
                c.rms_norm(kh, L["k_norm"], cfg.eps, kh)
                c.rope(qh, qh, T, cfg.heads, D, self.cos, self.sin, D, self.past, pos_dev)
                c.rope(kh, kh, T, cfg.kv_heads, D, self.cos, self.sin, D, self.past, pos_dev)
                c.attention(qh, kh, v, L["k_cache"], L["v_cache"], attn, T, cfg.heads,
                            cfg.kv_heads, D, self.past, self.capacity, D ** -0.5, pos_dev)
            c.matmul(L["o"], attn, o, rule=rule)
            c.add_rms_norm(x, o, L["ln2"], cfg.eps, h)       # x += o; h = norm(x)
            if cfg.experts:  # router, selection, expert matmuls and combine: one operator
                c.moe_forward(h, L["router"], cfg.top_k, cfg.intermediate, L["gate_up"],
                              L["down"], dn)
            else:
                c.matmul(L["gate_up"], h, gu, rule=rule)
                c.swiglu(gu, act)
                c.matmul(L["down"], act, dn, rule=rule)
            nxt = self.layers[li + 1]["ln1"] if li + 1 < len(self.layers) else self.final_norm
            c.add_rms_norm(x, dn, nxt, cfg.eps, h)           # x += dn; h = next norm(x)
        if on_device_position:  # history[past] = the token that went in; past += 1
            c.advance(self.past_dev, T, ids_dev, self.history)
        c.matmul_argmax(self.lm_head, h[T - 1:T], self.token)
        if not on_device_position:
            self.past += T

    def prefill(self, ids):
        ids_dev = self.torch.from_numpy(np.asarray(ids, dtype=np.int32)).to(self.device)
        self.forward(ids_dev, len(ids))
        self.past_dev.fill_(self.past)

    def decode_step(self):
        """One greedy step: the token chosen by the previous step goes in."""
        self.forward(self.token, 1)
        self.past_dev.fill_(self.past)

    def capture_decode_step(self):
        """Captures one decode step -- position, token in and token out all on the device --
        in a CUDA graph; replay_decode_step() then costs one graph launch per token."""
        torch = self.torch
        # one step outside the capture (first-use set-up of the kernels); the token and the
        # position are put back, and the cache row it wrote is the one the next step rewrites
        token = self.token.clone()
        self.past_dev.fill_(self.past)
        self.forward(self.token, 1, on_device_position=True)
        self.ctx.sync()
        self.token.copy_(token)
        self.past_dev.fill_(self.past)
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        main = torch.cuda.current_stream().cuda_stream
        with torch.cuda.stream(side):
            self.ctx.set_stream(side.cuda_stream)
            with torch.cuda.graph(g, stream=side):
                self.forward(self.token, 1, on_device_position=True)
        self.ctx.set_stream(main)
        self.step_graph = g

    def replay_decode_step(self):
        self.step_graph.replay()
        self.past += 1

    def generate(self, prompt_ids, steps, replay=False):
        """Greedy tokens: the one after the prompt and `steps - 1` more.  replay: the decode
        steps are replays of one captured graph with no host read in between; the tokens come
        back from the device's history at the end."""
        self.reset()
        self.prefill(prompt_ids)
        if replay:
            if self.step_graph is None:
                self.capture_decode_step()
            for _ in range(steps - 1):
                self.replay_decode_step()
            self.ctx.sync()
            self.torch.cuda.synchronize()
            n = len(prompt_ids)
            return self.history[n:n + steps - 1].cpu().tolist() + [int(self.token.item())]
        out = []
        for _ in range(steps):
            self.ctx.sync()
            out.append(int(self.token.item()))
            if len(out) < steps:
                self.decode_step()
        return out

    def free(self):
        for L in self.layers:
            for k in ("qkv", "o", "gate_up", "down"):
                L[k].free()
        self.lm_head.free()


class TensorParallelDecoder(DenseDecoder):
    """The decoder over `world` ranks (one process per GPU, torch.distributed): every
    matmul is split by output rows (shard.decoder_layer_shard), attention runs on the rank's
    own heads with a cache of their own, and the pieces are put together again by four
    all-gathers per layer -- after attention, o, SwiGLU and down -- so that every rank holds
    the full residual stream and the result is the one-GPU result bit for bit (row-split
    matmuls are exact; norms and residual adds run replicated).  A routed mixture of experts
    is split by expert instead (expert_parallel.ExpertParallelMoE: the rank's experts' route
    outputs, one all-reduce of the route buffer, the ordered combine on every rank).  The
    lm_head is split by rows too: every rank picks the best of its rows on the device and the
    (value, index) pairs are gathered; the largest value wins, the lowest index among equals,
    as on one GPU.

    Not run on GPUs yet: the class is exercised by world-size-2 gloo ranks on the CPU with the
    oracle standing in for the device operators (tests/test_tp_decoder_cpu.py), where its
    tokens are those of the one-rank decoder."""

    def __init__(self, ctx, cfg, weights, capacity, rank, world, group=None,
                 multi_row_rule=capi.ACT_G32, device="cuda"):
        import torch
        import torch.distributed as dist
        from . import shard
        if cfg.vocab % (8 * world):
            raise ValueError(f"vocabulary {cfg.vocab} does not split into 8-row tiles over "
                             f"{world} ranks")
        self.dist, self.group, self.rank, self.world = dist, group, rank, world
        self.full = cfg
        # what the base class sets up: this rank's heads, its slice of the intermediate
        # features (or its experts) and its slice of the vocabulary
        local = DecoderConfig(cfg.layers, cfg.hidden, cfg.heads // world, cfg.kv_heads // world,
                              cfg.head_dim,
                              cfg.intermediate if cfg.experts else cfg.intermediate // world,
                              cfg.vocab // world, rope_theta=cfg.rope_theta, eps=cfg.eps,
                              experts=cfg.experts // world if cfg.experts else 0,
                              top_k=cfg.top_k)
        sharded, local_shapes = [], None
        for layer in weights["layers"]:
            w, local_shapes = shard.decoder_layer_shard(cfg, weights["shapes"], layer, rank, world)
            sharded.append(w)
        v_lo, v_hi = shard.row_range(cfg.vocab, rank, world)
        local_weights = {"shapes": local_shapes, "layers": sharded,
                         "final_norm": weights["final_norm"], "embed": weights["embed"],
                         "lm_head": shard.rows_of(weights["lm_head"], cfg.hidden, v_lo, v_hi)}
        super().__init__(ctx, local, local_weights, capacity, multi_row_rule=multi_row_rule,
                         device=device)
        self.moe = []
        if cfg.experts:
            from .expert_parallel import DeviceEngine, ExpertParallelMoE
            e_lo, e_hi = shard.expert_range(cfg.experts, rank, world)
            reduce_sum = lambda t: dist.all_reduce(t, group=group)
            for L in self.layers:
                engine = DeviceEngine(ctx, L["router"], L["gate_up"], L["down"], cfg.top_k,
                                      cfg.intermediate, e_lo, e_hi - e_lo)
                self.moe.append(ExpertParallelMoE(engine, reduce_sum))
        self.vocab_offset = v_lo
        self.best = torch.zeros((2,), dtype=torch.float32, device=device)  # value, index
        self.logits = torch.zeros((1, local.vocab), dtype=torch.float32, device=device)
        self.local_token = torch.zeros((1,), dtype=torch.int32, device=device)

    def _gather_columns(self, local, name):
        """[T, n] per rank -> [T, world * n] on every rank, rank r's columns at r * n."""
        torch, T, n = self.torch, local.shape[0], local.shape[1]
        parts = self._b(name + "_parts", self.world * T, n).view(self.world, T, n)
        self.dist.all_gather([parts[p] for p in range(self.world)], local.contiguous(),
                             group=self.group)
        full = self._b(name + "_full", T, self.world * n)
        full.view(T, self.world, n).copy_(parts.permute(1, 0, 2))
        return full

    def forward(self, ids_dev, tokens, on_device_position=False):
        c, cfg, full = self.ctx, self.cfg, self.full
        T, H, D = tokens, full.hidden, full.head_dim
        rule = capi.ACT_G128 if T == 1 else self.multi_row_rule
        pos_dev = self.past_dev if on_device_position else None
        x, h = self._b("x", T, H), self._b("h", T, H)
        qkv = self._b("qkv", T, cfg.q_dim + 2 * cfg.kv_dim)
        q, attn_l = self._b("q", T, cfg.q_dim), self._b("attn", T, cfg.q_dim)
        o_l, dn_l = self._b("o", T, H // self.world), self._b("dn", T, H // self.world)
        gu = act_l = None
        if not full.experts:
            gu = self._b("gu", T, 2 * cfg.intermediate)
            act_l = self._b("act", T, cfg.intermediate)
        c.embed_rows(self.embed, ids_dev, x)
        c.rms_norm(x, self.layers[0]["ln1"], full.eps, h)
        for li, L in enumerate(self.layers):
            c.matmul(L["qkv"], h, qkv, rule=rule)
            c.qkv_prepare(qkv, T, cfg.heads, cfg.kv_heads, D, L["q_norm"], L["k_norm"], full.eps,
                          self.cos, self.sin, self.past, q, L["k_cache"], L["v_cache"],
                          self.capacity, pos_dev)
            c.attention(q, None, None, L["k_cache"], L["v_cache"], attn_l, T, cfg.heads,
                        cfg.kv_heads, D, self.past, self.capacity, D ** -0.5, pos_dev)
            attn = self._gather_columns(attn_l, "attn")        # [T, all heads * D]
            c.matmul(L["o"], attn, o_l, rule=rule)
            o = self._gather_columns(o_l, "o")                 # [T, H]
            c.add_rms_norm(x, o, L["ln2"], full.eps, h)
            if full.experts:  # the rank's experts, all-reduce of the route rows, combine
                dn = self.moe[li].forward(h, self._b("moe_out", T, H))
            else:
                c.matmul(L["gate_up"], h, gu, rule=rule)
                c.swiglu(gu, act_l)
                act = self._gather_columns(act_l, "act")       # [T, I]
                c.matmul(L["down"], act, dn_l, rule=rule)
                dn = self._gather_columns(dn_l, "dn")
            nxt = self.layers[li + 1]["ln1"] if li + 1 < len(self.layers) else self.final_norm
            c.add_rms_norm(x, dn, nxt, full.eps, h)
        if on_device_position:
            c.advance(self.past_dev, T, ids_dev, self.history)
        # the rank's best row (first maximum, as on one GPU) and its logit, then the best of all
        c.matmul_argmax(self.lm_head, h[T - 1:T], self.local_token, y=self.logits)
        torch = self.torch
        index = self.local_token.to(torch.int64)
        self.best[0] = self.logits[0].gather(0, index)[0]
        self.best[1] = (index[0] + self.vocab_offset).to(torch.float32)  # exact below 2^24
        pairs = self._b("best_parts", self.world, 2)
        self.dist.all_gather([pairs[p] for p in range(self.world)], self.best, group=self.group)
        top = pairs[:, 0].max()
        winners = torch.where(pairs[:, 0] == top, pairs[:, 1], torch.full_like(pairs[:, 1], 3e7))
        self.token.copy_(winners.min().to(torch.int32).reshape(1))
        if not on_device_position:
            self.past += T
