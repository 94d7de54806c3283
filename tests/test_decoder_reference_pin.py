"""The decoder against the REFERENCE'S OWN ENGINE.  tests/golden/tiny_qwen3_w4g128.mollm and
tiny_qwen3_moe_w4g128.mollm are two-layer Qwen3 packages (dense; 8 routed experts, 2 per token)
written by the reference's converter (models/converter.py, W4G128 through
tools/quantize_weight.cpp) and the *_reference.npz files hold what the reference's CPU engine
(LLMEngine::prefill / decode, greedy) answers on them; all come from
tests/golden/make_decoder_golden.py.

  * the package reader (palm-infra_b200/package.py) finds every weight the decoder needs;
  * the CPU decoder of the tests, with the exact product of fp32 activations and dequantised
    weights in place of W4A8 (the arithmetic of the reference's x86 build), reproduces the
    engine's logits to 1e-5 and all 32 greedy tokens: the decoder's structure -- fused qkv,
    per-head norms, rotary convention, cache and attention, SwiGLU, residuals, final norm,
    lm_head -- is the reference's;
  * with W4A8 (the arithmetic of the GPU path and of the reference's ARM build) the logits sit
    within the activation-quantisation distance of the engine's and the tokens are the same
    (the fixture's seed was chosen for margins above that distance);
  * against the engine run with the W4A8 matmul at its provider seam
    (kernels/cpu_platform.h:75-79; oracle/ref_shim.cpp) -- the reference's graph executor,
    norms, rotary embedding, attention, MoE control flow and sampler around the restated
    matmul -- the dense CPU decoder is identical BIT FOR BIT, logits and tokens, on the
    recorded run and, where the reference library is present, live on prompts of many
    lengths; with routed experts the logits agree to a few ulp (2e-6) and the tokens exactly:
    the engine's x86 build takes the router's fp16 matmul and the weighted sum of the expert
    outputs in another order than its ARM build, which the oracle follows by default -- and
    when the oracle is told to take those two sums the x86 way (ol.set_moe_host_build), that
    decoder is bit-identical to the engine as well, so these two sums are the whole difference;
  * (gpu) the device decoder gives the engine's tokens too, eager and replayed.
"""
import os

import numpy as np
import pytest

import oracle_lib as ol
from golden_util import rel_l2
from __graft_entry__ import load_package

pkg = load_package()
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_fixture(stem):
    path = os.path.join(GOLDEN, stem + "_w4g128.mollm")
    package = pkg.package.read_package(path)
    package.path = path
    cfg, weights = pkg.package.qwen3_decoder_weights(package)
    ref = np.load(os.path.join(GOLDEN, stem + "_reference.npz"))
    package.w4a8 = (ref["tokens_w4a8"].tolist(), ref["logits_w4a8"])
    return package, cfg, weights, ref["prompt"].tolist(), ref["tokens"].tolist(), ref["logits"]


@pytest.fixture(scope="module", params=["tiny_qwen3", "tiny_qwen3_moe"])
def fixture(request):
    return load_fixture(request.param)


def test_package_reader_finds_the_decoder(fixture):
    package, cfg, weights, *_ = fixture
    assert package.metadata["architecture"] in ("qwen3", "qwen3-moe")
    assert package.metadata["quantization"] == "w4g128"
    assert (cfg.layers, cfg.hidden, cfg.heads, cfg.kv_heads, cfg.head_dim) == (2, 256, 4, 2, 64)
    assert cfg.vocab == 512 and cfg.rope_theta == 1e6
    if cfg.experts:
        assert (cfg.experts, cfg.top_k, cfg.intermediate) == (8, 2, 128)
        assert all(layer["router"].shape == (8, 256) for layer in weights["layers"])
    else:
        assert cfg.intermediate == 512
    assert weights["embed"].shape == (512, 256) and weights["embed"].dtype == np.float16
    assert weights["lm_head"].size == ol.bg128_bytes(512, 256)
    for layer in weights["layers"]:
        for key, (n, k) in weights["shapes"].items():
            assert layer[key].size == ol.bg128_bytes(n, k)
    with pytest.raises(pkg.package.PackageError):
        package.weight("no_such_weight.weights")


def test_exact_arithmetic_reproduces_the_reference_engine(fixture):
    _, cfg, weights, prompt, tokens, logits = fixture
    first = []
    got, _ = ol.dense_decoder_tokens(cfg, weights, prompt, len(tokens), every_rule=ol.ACT_F64,
                                     first_logits=first)
    assert rel_l2(first[0], logits) < 1e-5
    assert got == tokens


def test_w4a8_tokens_are_the_reference_engines(fixture):
    _, cfg, weights, prompt, tokens, logits = fixture
    first = []
    ol.set_exp_mode(True)  # exp as the device takes it; the tokens do not depend on it here
    try:
        got, margins = ol.dense_decoder_tokens(cfg, weights, prompt, len(tokens),
                                               first_logits=first)
    finally:
        ol.set_exp_mode(False)
    assert rel_l2(first[0], logits) < 3e-2  # W4A8 against W4A32: the activation quantisation
    assert got == tokens
    assert min(margins) > 1e-2


def test_w4a8_decoder_is_the_engine_with_the_w4a8_provider_bit_for_bit(fixture):
    package, cfg, weights, prompt, tokens, _ = fixture
    engine_tokens, engine_logits = package.w4a8
    first = []
    got, _ = ol.dense_decoder_tokens(cfg, weights, prompt, len(tokens), first_logits=first)
    if cfg.experts:
        assert rel_l2(first[0], engine_logits) < 2e-6
        ol.set_moe_host_build(True)  # the fixture was recorded with the x86 build
        try:
            again = []
            got_x86, _ = ol.dense_decoder_tokens(cfg, weights, prompt, len(tokens),
                                                 first_logits=again)
        finally:
            ol.set_moe_host_build(False)
        assert again[0].tobytes() == engine_logits.tobytes()
        assert got_x86 == engine_tokens
    else:
        assert first[0].tobytes() == engine_logits.tobytes()
    assert got == engine_tokens


@pytest.mark.skipif(not ol.have_ref(), reason="the reference library is not built")
def test_live_engine_with_the_w4a8_provider_on_other_prompts(fixture):
    """The committed package through the live reference engine, prompts of several lengths
    (one token: every matmul of the prompt takes the one-row rule)."""
    package, cfg, weights, *_ = fixture
    for length in (1, 2, 3, 5, 8, 17, 40):
        prompt = np.random.default_rng(200 + length).integers(0, cfg.vocab, length).tolist()
        engine_tokens, engine_logits = ol.ref_engine_generate(package.path, prompt, 6,
                                                              cfg.vocab, w4a8=True)
        first = []
        got, margins = ol.dense_decoder_tokens(cfg, weights, prompt, 6, first_logits=first)
        if cfg.experts:
            assert rel_l2(first[0], engine_logits) < 2e-6, length
            ol.set_moe_host_build(True)  # this host's build of the reference is the x86 one
            try:
                again = []
                got_x86, _ = ol.dense_decoder_tokens(cfg, weights, prompt, 6,
                                                     first_logits=again)
            finally:
                ol.set_moe_host_build(False)
            assert again[0].tobytes() == engine_logits.tobytes(), length
            assert got_x86 == engine_tokens, length
        else:
            assert first[0].tobytes() == engine_logits.tobytes(), length
        if min(margins) > 1e-4:  # a few ulp cannot turn a token with such a margin
            assert got == engine_tokens, length
    # and the unmodified engine still is what the fixture recorded
    recorded = np.load(os.path.join(GOLDEN, os.path.basename(package.path).replace(
        "_w4g128.mollm", "_reference.npz")))
    live, _ = ol.ref_engine_generate(package.path, recorded["prompt"].tolist(),
                                     len(recorded["tokens"]), cfg.vocab)
    assert live == recorded["tokens"].tolist()


def test_decoder_driver_gives_the_reference_engines_tokens_on_the_cpu(fixture):
    """palm-infra_b200/decoder.py itself -- the operator sequence, buffers and cache handling
    that run on the GPU -- with the oracle standing in for the device operators."""
    from cpu_context import OracleContext
    _, cfg, weights, prompt, tokens, _ = fixture
    model = pkg.decoder.DenseDecoder(OracleContext(), cfg, weights,
                                     capacity=len(prompt) + len(tokens) + 8, device="cpu")
    ol.set_exp_mode(True)
    try:
        assert model.generate(prompt, len(tokens)) == tokens
    finally:
        ol.set_exp_mode(False)


@pytest.mark.gpu
def test_device_decoder_gives_the_reference_engines_tokens(fixture):
    _, cfg, weights, prompt, tokens, _ = fixture
    ctx = pkg.capi.Context(0)
    model = pkg.decoder.DenseDecoder(ctx, cfg, weights, capacity=len(prompt) + len(tokens) + 8)
    eager = model.generate(prompt, len(tokens))
    replayed = model.generate(prompt, len(tokens), replay=True)
    model.free()
    ctx.close()
    assert eager == tokens == fixture[0].w4a8[0]
    assert replayed == tokens
