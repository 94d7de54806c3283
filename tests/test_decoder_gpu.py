"""A Qwen3-shaped dense decoder end to end on the GPU (palm-infra_b200/decoder.py: every
operator a libb200w4 kernel) against the same decoder computed on the CPU from the oracle's
pieces: greedy tokens must be identical over a prompt and a run of decode steps, with the
reference's activation rule (per 128 values for one row, per 32 for the prompt's rows).  The
matmuls are bit-exact on both sides; the norms, the attention scores and the softmax differ by
the rounding of reassociated fp32 sums, so identity rests on the top-1 margins, which the test
prints and requires to be far above that noise."""
import numpy as np
import pytest

import oracle_lib as ol
from __graft_entry__ import load_package

pkg = load_package()
pytestmark = pytest.mark.gpu


# Seeds are chosen on the CPU (the oracle decoder alone) for a comfortable smallest top-1 margin
# over the run: 5e-2 for the 64-step case.
@pytest.mark.parametrize("layers,hidden,heads,kv_heads,head_dim,inter,vocab,prompt_len,steps,"
                         "seed",
                         [(2, 256, 4, 2, 64, 512, 1000, 12, 64, 11),   # 64 greedy steps
                          (3, 512, 8, 2, 128, 1024, 2048, 33, 16, 20261128),
                          # benchmark configuration 3's widths (hidden 2560, 32 / 8 heads of 128,
                          # intermediate 9728, vocabulary 151936) at four layers: what the CPU
                          # decoder finishes in about a minute
                          (4, 2560, 32, 8, 128, 9728, 151936, 8, 6, 20261129)])
def test_greedy_tokens_identical_to_the_cpu_decoder(layers, hidden, heads, kv_heads, head_dim,
                                                   inter, vocab, prompt_len, steps, seed):
    dec = pkg.decoder
    cfg = dec.DecoderConfig(layers, hidden, heads, kv_heads, head_dim, inter, vocab)
    weights = dec.synthetic_weights(cfg, seed=seed)
    prompt = np.random.default_rng(11).integers(0, vocab, prompt_len).tolist()
    ol.set_exp_mode(True)
    try:
        want, margins = ol.dense_decoder_tokens(cfg, weights, prompt, steps)
    finally:
        ol.set_exp_mode(False)
    ctx = pkg.capi.Context(0)
    model = dec.DenseDecoder(ctx, cfg, weights, capacity=prompt_len + steps + 8)
    got = model.generate(prompt, steps)
    replayed = model.generate(prompt, steps, replay=True)  # one captured step, replayed
    model.free()
    model = dec.DenseDecoder(ctx, cfg, weights, capacity=prompt_len + steps + 8, fused_qkv=False)
    unfused = model.generate(prompt, steps)                # operator by operator
    model.free()
    ctx.close()
    print(f"tokens {got}\nminimum top-1 margin {min(margins):.3e}")
    assert got == want, (got, want, margins)
    assert replayed == want, (replayed, want)
    assert unfused == want, (unfused, want)
    assert min(margins) > 1e-2  # identity is not an accident of a near-tie


@pytest.mark.parametrize("layers,hidden,heads,kv_heads,head_dim,inter,vocab,experts,top_k,"
                         "prompt_len,steps,seed",
                         [(2, 256, 4, 2, 64, 128, 1000, 8, 2, 12, 64, 4),   # 64 greedy steps
                          # benchmark configuration 4's widths (hidden 2048, 32 / 4 heads of 128,
                          # 128 experts of width 768, 8 per token) at two layers
                          (2, 2048, 32, 4, 128, 768, 4096, 128, 8, 20, 6, 77 + 128)])
def test_mixture_of_experts_decoder_tokens_identical(layers, hidden, heads, kv_heads, head_dim,
                                                    inter, vocab, experts, top_k, prompt_len,
                                                    steps, seed):
    """The same identity with the MOE operator as the feed-forward block (router, selection,
    expert matmuls under the reference's per-expert activation rule, ordered combine): prompt
    rows give experts several rows each, decode steps one."""
    dec = pkg.decoder
    cfg = dec.DecoderConfig(layers, hidden, heads, kv_heads, head_dim, inter, vocab,
                            experts=experts, top_k=top_k)
    weights = dec.synthetic_weights(cfg, seed=seed)
    prompt = np.random.default_rng(5).integers(0, vocab, prompt_len).tolist()
    ol.set_exp_mode(True)
    try:
        want, margins = ol.dense_decoder_tokens(cfg, weights, prompt, steps)
    finally:
        ol.set_exp_mode(False)
    ctx = pkg.capi.Context(0)
    model = dec.DenseDecoder(ctx, cfg, weights, capacity=prompt_len + steps + 8)
    got = model.generate(prompt, steps)
    replayed = model.generate(prompt, steps, replay=True)
    model.free()
    ctx.close()
    print(f"tokens {got}\nminimum top-1 margin {min(margins):.3e}")
    assert got == want, (got, want, margins)
    assert replayed == want, (replayed, want)
    assert min(margins) > 1e-2
