#!/usr/bin/env python3
"""Generates the decoder fixtures: tiny Qwen3 model packages (one dense, one with routed
experts) made by the REFERENCE's own converter, and what the REFERENCE's own CPU engine answers
on them.

    python tests/golden/make_decoder_golden.py [dense seed] [mixture-of-experts seed]

Needs the reference tree (environment variable REF_ROOT) and `make -C oracle ref reftools`;
it is run where the reference is available, and its outputs are committed:

    tests/golden/tiny_qwen3_w4g128.mollm        the dense package (about 1 MB)
    tests/golden/tiny_qwen3_reference.npz       prompt, the engine's greedy tokens and the
                                                logits of the prompt's last position, as the
                                                x86 build computes them (W4A32) and with the
                                                W4A8 matmul at the engine's provider seam
    tests/golden/tiny_qwen3_moe_w4g128.mollm, tiny_qwen3_moe_reference.npz
                                                the same for 8 experts of width 128, 2 per token

Steps, all with reference code: a Hugging-Face-style directory with seeded random weights
(config.json + model.safetensors, the fixture recipe of tests/run_tiny_qwen3_cpu_e2e.py scaled
up to widths that W4G128 accepts) -> models/converter.py with quantisation w4g128 (which calls
tools/quantize_weight.cpp, built as oracle/_ref/mollm-quantize) -> LLMEngine on the CPU, greedy
(oracle/ref_shim.cpp `ref_engine_generate`).

The reference's x86 build multiplies fp32 activations with dequantised weights (W4A32); the
W4A8 decoders of this repository differ from it by the activation quantisation, so the seed is
chosen for top-1 margins far above that difference (printed below), and the tests compare
those logits with a tolerance and the tokens exactly.  The second recording runs the same
engine with its INT4 matmuls answered, at the provider seam the reference documents
(kernels/cpu_platform.h:75-79), by the oracle's W4A8 arithmetic under the reference's rule per
row count (oracle/ref_shim.cpp): what the reference's ARM build computes, with every other
operator the reference's own code.  Against that recording the comparison is bit for bit.
"""
import ctypes as C
import json
import os
import shutil
import struct
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
REF_ROOT = Path(os.environ.get("REF_ROOT", "/root/reference"))
REF_DIR = ROOT / "oracle" / "_ref"

LAYERS, HIDDEN, HEADS, KV_HEADS, HEAD_DIM, INTER, VOCAB = 2, 256, 4, 2, 64, 512, 512
EXPERTS, TOP_K, MOE_INTER = 8, 2, 128
PROMPT_LEN, STEPS = 12, 32


def write_safetensors(path, tensors):
    header, parts, offset = {}, [], 0
    for name, array in tensors.items():
        array = np.ascontiguousarray(array)
        dtype = {"float16": "F16", "float32": "F32"}[str(array.dtype)]
        payload = array.tobytes()
        header[name] = {"dtype": dtype, "shape": list(array.shape),
                        "data_offsets": [offset, offset + len(payload)]}
        parts.append(payload)
        offset += len(payload)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    Path(path).write_bytes(struct.pack("<Q", len(encoded)) + encoded + b"".join(parts))


def build_model_dir(model_dir, seed, experts=0):
    rng = np.random.default_rng(seed)

    def matrix(rows, cols, std=0.05):
        return (rng.standard_normal((rows, cols)) * std).astype(np.float16)

    def norm(n):
        return (1.0 + 0.05 * rng.standard_normal(n)).astype(np.float32)

    config = {"model_type": "qwen3", "hidden_size": HIDDEN, "num_hidden_layers": LAYERS,
              "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "num_attention_heads": HEADS,
              "num_key_value_heads": KV_HEADS, "head_dim": HEAD_DIM,
              "intermediate_size": INTER, "vocab_size": VOCAB}
    if experts:  # the fields models/qwen3_moe.py reads (softmax routing, weights renormalised)
        config.update({"model_type": "qwen3_moe", "moe_intermediate_size": MOE_INTER,
                       "num_experts": experts, "num_experts_per_tok": TOP_K,
                       "norm_topk_prob": True, "decoder_sparse_step": 1, "mlp_only_layers": []})
    (model_dir / "config.json").write_text(json.dumps(config), encoding="utf-8")
    tensors = {"model.embed_tokens.weight": matrix(VOCAB, HIDDEN, 0.5),
               "lm_head.weight": matrix(VOCAB, HIDDEN), "model.norm.weight": norm(HIDDEN)}
    for l in range(LAYERS):
        p = f"model.layers.{l}"
        tensors.update({
            f"{p}.input_layernorm.weight": norm(HIDDEN),
            f"{p}.post_attention_layernorm.weight": norm(HIDDEN),
            f"{p}.self_attn.q_proj.weight": matrix(HEADS * HEAD_DIM, HIDDEN),
            f"{p}.self_attn.k_proj.weight": matrix(KV_HEADS * HEAD_DIM, HIDDEN),
            f"{p}.self_attn.v_proj.weight": matrix(KV_HEADS * HEAD_DIM, HIDDEN),
            f"{p}.self_attn.q_norm.weight": norm(HEAD_DIM),
            f"{p}.self_attn.k_norm.weight": norm(HEAD_DIM),
            f"{p}.self_attn.o_proj.weight": matrix(HIDDEN, HEADS * HEAD_DIM)})
        if experts:
            tensors[f"{p}.mlp.gate.weight"] = matrix(experts, HIDDEN, 0.5)
            for e in range(experts):
                tensors.update({
                    f"{p}.mlp.experts.{e}.gate_proj.weight": matrix(MOE_INTER, HIDDEN),
                    f"{p}.mlp.experts.{e}.up_proj.weight": matrix(MOE_INTER, HIDDEN),
                    f"{p}.mlp.experts.{e}.down_proj.weight": matrix(HIDDEN, MOE_INTER)})
        else:
            tensors.update({
                f"{p}.mlp.gate_proj.weight": matrix(INTER, HIDDEN),
                f"{p}.mlp.up_proj.weight": matrix(INTER, HIDDEN),
                f"{p}.mlp.down_proj.weight": matrix(HIDDEN, INTER)})
    write_safetensors(model_dir / "model.safetensors", tensors)


def convert(model_dir, package):
    env = dict(os.environ, MOLLM_QUANT_HELPER=str(REF_DIR / "mollm-quantize"),
               MOLLM_QUANT_THREADS="1")
    subprocess.run([sys.executable, str(REF_ROOT / "models" / "converter.py"), str(model_dir),
                    str(package), "w4g128"], check=True, env=env, cwd=str(REF_ROOT),
                   stdout=subprocess.DEVNULL)


def reference_engine(package, prompt, steps, w4a8=False):
    lib = C.CDLL(str(REF_DIR / "libref_shim.so"))
    lib.ref_set_w4a8_provider(1 if w4a8 else 0)
    ids = np.asarray(prompt, dtype=np.int32)
    tokens = np.zeros(steps, dtype=np.int32)
    logits = np.zeros(VOCAB, dtype=np.float32)
    rc = lib.ref_engine_generate(str(package).encode(), ids.ctypes.data_as(C.c_void_p), len(ids),
                                 steps, 256, 1, tokens.ctypes.data_as(C.c_void_p),
                                 logits.ctypes.data_as(C.c_void_p), VOCAB)
    lib.ref_set_w4a8_provider(0)
    if rc != 0:
        raise RuntimeError(f"ref_engine_generate returned {rc}")
    return tokens, logits


def make(seed, experts, stem):
    tmp = Path(tempfile.mkdtemp(prefix="decoder_golden_"))
    try:
        model_dir = tmp / "model"
        model_dir.mkdir()
        build_model_dir(model_dir, seed, experts)
        package = tmp / "tiny.mollm"
        convert(model_dir, package)
        prompt = np.random.default_rng(seed + 1).integers(0, VOCAB, PROMPT_LEN).astype(np.int32)
        tokens, logits = reference_engine(package, prompt, STEPS)
        tokens_w4a8, logits_w4a8 = reference_engine(package, prompt, STEPS, w4a8=True)
        top = np.sort(logits)[-2:]
        print(f"{stem}, seed {seed}: reference tokens {tokens.tolist()}")
        print(f"top-1 margin at the prompt's end {top[1] - top[0]:.4f}, "
              f"logit scale {np.abs(logits).max():.3f}")
        shutil.copyfile(package, HERE / f"{stem}_w4g128.mollm")
        np.savez(HERE / f"{stem}_reference.npz", prompt=prompt, tokens=tokens, logits=logits,
                 tokens_w4a8=tokens_w4a8, logits_w4a8=logits_w4a8, seed=np.int64(seed))
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def main():
    dense_seed = int(sys.argv[1]) if len(sys.argv) > 1 else 24
    moe_seed = int(sys.argv[2]) if len(sys.argv) > 2 else 34
    if dense_seed >= 0:
        make(dense_seed, 0, "tiny_qwen3")
    if moe_seed >= 0:
        make(moe_seed, EXPERTS, "tiny_qwen3_moe")


if __name__ == "__main__":
    main()
