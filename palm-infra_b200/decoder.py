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
    all in fp32."""
    half = rope_dim // 2
    i = np.arange(half, dtype=np.float32)
    inv = (np.float32(1.0) / np.power(np.float32(theta), np.float32(2.0) * i / np.float32(rope_dim))
           ).astype(np.float32)
    ang = (np.asarray(positions, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


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
    def __init__(self, ctx, cfg, weights, capacity, multi_row_rule=capi.ACT_G32, fused_qkv=None):
        import torch
        self.torch, self.ctx, self.cfg, self.capacity = torch, ctx, cfg, capacity
        self.multi_row_rule = multi_row_rule
        can_fuse = cfg.head_dim % 64 == 0 and cfg.head_dim <= 256
        self.fused_qkv = can_fuse if fused_qkv is None else (fused_qkv and can_fuse)
        sh = weights["shapes"]
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        self.layers = []
        for w in weights["layers"]:
            self.layers.append({
                **{k: ctx.upload_weight(w[k], *sh[k]) for k in sh},
                **{k: dev(w[k]) for k in ("ln1", "ln2", "q_norm", "k_norm")},
                **({"router": dev(w["router"].view(np.int16))} if cfg.experts else {}),
                "k_cache": torch.zeros((cfg.kv_heads, capacity, cfg.head_dim), device="cuda"),
                "v_cache": torch.zeros((cfg.kv_heads, capacity, cfg.head_dim), device="cuda")})
        self.final_norm = dev(weights["final_norm"])
        self.embed = dev(weights["embed"].view(np.int16))
        self.lm_head = ctx.upload_weight(weights["lm_head"], cfg.vocab, cfg.hidden)
        cos, sin = rope_tables(range(capacity), cfg.head_dim, cfg.rope_theta)
        self.cos, self.sin = dev(cos), dev(sin)  # rows = positions
        self.past = 0
        self.token = torch.zeros((1,), dtype=torch.int32, device="cuda")
        self.past_dev = torch.zeros((1,), dtype=torch.int32, device="cuda")
        self.history = torch.zeros((capacity,), dtype=torch.int32, device="cuda")
        self.step_graph = None
        self._buf = {}

    def _b(self, name, rows, cols):
        key = (name, rows, cols)
        if key not in self._buf:
            self._buf[key] = self.torch.empty((rows, cols), dtype=self.torch.float32,
                                              device="cuda")
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
        ids_dev = self.torch.from_numpy(np.asarray(ids, dtype=np.int32)).cuda()
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
