"""Reader for the reference's single-file model package (`.mollm`), as far as a Qwen3-shaped
decoder (dense, or with the routed mixture of experts in every layer) with W4G128 weights
needs it: the package header and its JSON section
(written by models/transpile.py:1937 `save_package`, read by engine/package.cpp:216-279), the
weight files inside the weights region (88-byte header + payload, models/transpile.py:1460-1475;
INT4 tensors are canonical BG128 blocks with embedded scales, :1778-1830) and the key/value
section at the head of a graph file (models/transpile.py:1214-1226), where the converter puts
the rotary-embedding parameters the engine reads (engine/model_loader.cpp:1281-1282).

`qwen3_decoder_weights` turns a package into the configuration and weight dictionary that
`decoder.DenseDecoder` (and the CPU decoder of the tests) take, so a package produced by the
reference's own converter runs here unchanged.  Tokenizer, chat template and the graphs
themselves are not interpreted: the decoder's structure is fixed (models/qwen3.py:171-345).
"""
import json
import struct

import numpy as np

PACKAGE_MAGIC = 0x4D4C4F4D   # "MOLM"
WEIGHT_MAGIC = 0x50414D58    # "XMAP"
GRAPH_SECTION = {"prefill": 56, "decode": 72}  # (offset, length) pairs in the package header
_WEIGHT_HEADER = struct.Struct("<IIIIQQQQQQQQII")  # 88 bytes
FLAG_INT4_BG128 = 1 << 1
PREC_FP32, PREC_FP16, PREC_INT4 = 0, 1, 3


class PackageError(ValueError):
    pass


class PackedWeight:
    """One weight file of the package: logical shape, precision, storage flags, payload."""

    def __init__(self, name, flags, precision, shape, group_size, payload):
        self.name, self.flags, self.precision = name, flags, precision
        self.shape, self.group_size, self.payload = shape, group_size, payload

    def fp32(self):
        if self.precision != PREC_FP32:
            raise PackageError(f"{self.name}: precision {self.precision}, expected fp32")
        return np.frombuffer(self.payload, dtype=np.float32).copy()

    def fp16(self):
        if self.precision != PREC_FP16:
            raise PackageError(f"{self.name}: precision {self.precision}, expected fp16")
        return np.frombuffer(self.payload, dtype=np.float16).reshape(self.shape).copy()

    def bg128_blocks(self):
        """The canonical BG128 blocks of an INT4 [N, K] weight (544 bytes per 8 rows x 128 k),
        the bytes `b2w4_weight_upload` takes."""
        n, k = self.shape
        if self.precision != PREC_INT4 or not self.flags & FLAG_INT4_BG128 or \
                self.group_size != 128 or k % 128 or n % 8:
            raise PackageError(f"{self.name}: not a W4G128 BG128 weight with whole 8-row tiles")
        want = (n // 8) * (k // 128) * 544
        if len(self.payload) != want:
            raise PackageError(f"{self.name}: {len(self.payload)} payload bytes, expected {want}")
        return np.frombuffer(self.payload, dtype=np.uint8).copy()


class Package:
    def __init__(self, metadata, graph_metadata, weights):
        self.metadata, self.graph_metadata, self.weights = metadata, graph_metadata, weights

    def weight(self, name):
        for key in (name, "./" + name):
            if key in self.weights:
                return self.weights[key]
        raise PackageError(f"the package holds no weight named {name}")


def _graph_key_values(blob):
    """The key=value strings at the head of a graph file: magic, version, node count, pair
    count, then (length, bytes) twice per pair."""
    if len(blob) < 16:
        return {}
    count = struct.unpack_from("<I", blob, 12)[0]
    at, out = 16, {}
    for _ in range(count):
        pair = []
        for _ in range(2):
            n = struct.unpack_from("<I", blob, at)[0]
            pair.append(blob[at + 4:at + 4 + n].decode("utf-8"))
            at += 4 + n
        out[pair[0]] = pair[1]
    return out


def read_package(path):
    with open(path, "rb") as f:
        data = f.read()
    if len(data) < 128 or struct.unpack_from("<I", data, 0)[0] != PACKAGE_MAGIC:
        raise PackageError(f"{path}: not a .mollm package")
    meta_off, meta_len = struct.unpack_from("<QQ", data, 8)
    w_off, w_len = struct.unpack_from("<QQ", data, 88)
    metadata = json.loads(data[meta_off:meta_off + meta_len])
    g_off, g_len = struct.unpack_from("<QQ", data, GRAPH_SECTION["decode"])
    graph_metadata = _graph_key_values(data[g_off:g_off + g_len])
    weights = {}
    for name, (rel, size) in metadata.get("weights", {}).items():
        base = w_off + rel
        if size < _WEIGHT_HEADER.size or base + size > w_off + w_len:
            raise PackageError(f"{name}: weight range outside the weights region")
        (magic, flags, ndim, prec, s0, s1, s2, s3, d_off, d_size, _so, _ss, group,
         _groups) = _WEIGHT_HEADER.unpack_from(data, base)
        if magic != WEIGHT_MAGIC:
            raise PackageError(f"{name}: bad weight magic 0x{magic:08x}")
        shape = tuple(int(v) for v in (s0, s1, s2, s3)[:ndim])
        weights[name] = PackedWeight(name, flags, prec, shape, group,
                                     data[base + d_off:base + d_off + d_size])
    return Package(metadata, graph_metadata, weights)


def qwen3_decoder_weights(package):
    """(DecoderConfig, weights) of a Qwen3 package with W4G128 matmul weights, dense
    (architecture "qwen3") or with softmax-routed experts in every layer ("qwen3-moe", no shared
    expert, no dense head layers).  Names as the reference's converters write them
    (models/qwen3.py:171-345, models/qwen3_moe.py:337-520): fused qkv and gate_up projections,
    expert aggregates [E * 2I, H] and [E * H, I] with expert e's rows together, fp16 embedding
    and router rows, fp32 norms."""
    from .decoder import DecoderConfig
    m = package.metadata
    arch = m.get("architecture")
    if arch not in ("qwen3", "qwen3-moe"):
        raise PackageError(f"architecture {arch!r}: only qwen3 and qwen3-moe are read")
    layers, hidden = int(m["num_layers"]), int(m["hidden_size"])
    heads, kv_heads, head_dim = int(m["num_heads"]), int(m["num_kv_heads"]), int(m["head_dim"])
    vocab = int(m["vocab_size"])
    experts = top_k = 0
    if arch == "qwen3-moe":
        experts, top_k = int(m["num_experts"]), int(m["num_experts_per_tok"])
        if int(m.get("first_k_dense_replace", 0)) or int(m.get("n_shared_experts", 0)):
            raise PackageError("dense head layers and shared experts are not read")
        inter = int(m["moe_intermediate_size"])
    else:
        inter = package.weight("model_layers_0_mlp_gate_up_proj_weight.weights").shape[0] // 2
    theta = float(package.graph_metadata.get("rope_theta", 1e6))
    rope_dim = int(package.graph_metadata.get("rope_dim", head_dim))
    if rope_dim != head_dim:
        raise PackageError(f"rope over {rope_dim} of {head_dim} features is not supported here")
    cfg = DecoderConfig(layers, hidden, heads, kv_heads, head_dim, inter, vocab, rope_theta=theta,
                        eps=float(package.graph_metadata.get("rms_norm_eps", 1e-6)),
                        experts=experts, top_k=top_k)
    per = max(1, experts)
    shapes = {"qkv": (cfg.q_dim + 2 * cfg.kv_dim, hidden), "o": (hidden, cfg.q_dim),
              "gate_up": (per * 2 * inter, hidden), "down": (per * hidden, inter)}
    names = {"qkv": "self_attn_qkv_proj_weight", "o": "self_attn_o_proj_weight",
             "gate_up": "mlp_experts_gate_up_proj" if experts else "mlp_gate_up_proj_weight",
             "down": "mlp_experts_down_proj" if experts else "mlp_down_proj_weight",
             "ln1": "input_layernorm_weight", "ln2": "post_attention_layernorm_weight",
             "q_norm": "self_attn_q_norm_weight", "k_norm": "self_attn_k_norm_weight"}
    out_layers = []
    for l in range(layers):
        w = {}
        for key, tail in names.items():
            pw = package.weight(f"model_layers_{l}_{tail}.weights")
            if key in shapes:
                if pw.shape != shapes[key]:
                    raise PackageError(f"{pw.name}: shape {pw.shape}, expected {shapes[key]}")
                w[key] = pw.bg128_blocks()
            else:
                w[key] = pw.fp32()
        if experts:
            router = package.weight(f"model_layers_{l}_mlp_gate_weight.weights").fp16()
            if router.shape != (experts, hidden):
                raise PackageError(f"layer {l}: router shape {router.shape}")
            w["router"] = router
        out_layers.append(w)
    lm_head = package.weight("lm_head.weights")
    if lm_head.shape != (vocab, hidden):
        raise PackageError(f"lm_head: shape {lm_head.shape}")
    return cfg, {"shapes": shapes, "layers": out_layers,
                 "final_norm": package.weight("final_norm.weights").fp32(),
                 "embed": package.weight("embed_tokens.weights").fp16(),
                 "lm_head": lm_head.bg128_blocks()}
