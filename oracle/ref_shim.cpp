// Test infrastructure only: a thin extern "C" window onto the UNMODIFIED
// reference CPU library (compiled by oracle/Makefile into
// oracle/_ref/libmollm_ref.so).  It exists so that tests, the fixture
// generator and the bench's CPU-baseline leg can call the reference's own
// functions through ctypes.  No arithmetic happens here: every function builds
// the reference's Tensor descriptors and forwards.
//
// Reference entry points that are forwarded to:
//   quantize_a_q8_g128_even_odd   kernels/matmul_quant.cpp:578-641
//   quantize_a_q8_blocks          kernels/matmul_quant.cpp:280-329
//   kernel_matmul_fp32            kernels/matmul.cpp:69-97 (x86: W4A32 provider,
//                                 kernels/cpu_platform_x86.cpp:128-270)
//   pack_b_q4dot_int4_full / pack_b_q4dot_g128_full
//                                 kernels/matmul_pack.cpp:641-688
//   select_moe_routes             kernels/moe_routing.cpp:25-169
//   kernel_qwen3_moe              kernels/moe.cpp:576-1129
//   sample_token (temperature 0)  engine/sampler.cpp:458-462 -> argmax_token :31-77
//   kernel_rms_norm / kernel_add_rms_norm   kernels/norm.cpp:95-190
//   kernel_elementwise (SWIGLU)   kernels/elementwise.cpp:529-...
//   kernel_rope                   kernels/rope.cpp:155-195
//   sdpa_x86_avx512_head          kernels/attention_x86_avx512.cpp:47-109
//   LLMEngine::load / prefill / decode / prefill_hidden / run_lmhead_raw
//                                 engine/engine.h:170-330 (the whole CPU engine on a .mollm
//                                 package, as tests/test_tiny_cpu_inference.cpp drives it)
#include "kernels/attention_x86.h"
#include "kernels/elementwise.h"
#include "kernels/matmul.h"
#include "kernels/norm.h"
#include "kernels/rope.h"
#include "kernels/matmul_internal.h"
#include "kernels/moe.h"
#include "kernels/moe_routing.h"
#include "kernels/quant_layouts.h"
#include "kernels/threading.h"
#include "engine/engine.h"
#include "engine/sampler.h"
#include "kernels/cpu_platform.h"

#include <dlfcn.h>

#include <chrono>
#include <cstdint>
#include <cstring>
#include <memory>
#include <vector>

namespace {

Tensor make_bg128_weight(const void* blocks, int n, int k) {
    Tensor w = Tensor::create(Precision::INT4, MemoryType::EXTERNAL, n, k, 1, 1,
                              const_cast<void*>(blocks));
    w.group_size = 128;
    w.groups_per_row = static_cast<uint32_t>(k / 128);
    w.num_groups = static_cast<uint32_t>(n) * w.groups_per_row;
    w.is_q4_g128_packed = true;
    w.q4_g128_data = blocks;
    return w;
}

ThreadPool* pool_for(int threads) {
    static std::unique_ptr<ThreadPool> pool;
    static int pool_threads = 0;
    if (threads <= 1)
        return nullptr;
    if (!pool || pool_threads != threads) {
        pool.reset(new ThreadPool(threads));
        pool_threads = threads;
    }
    return pool.get();
}

}  // namespace

extern "C" {

const char* ref_isa_name() { return mollm::cpu::isa_name(); }

// M=1 activation quantiser, one scale per 128 values, even/odd de-interleaved.
void ref_quantize_a_q8_g128_even_odd(const float* a, int k, int8_t* even,
                                     int8_t* odd, float* scales) {
    std::vector<int8_t> e, o;
    std::vector<float> s;
    quantize_a_q8_g128_even_odd(a, k, e, o, s);
    std::memcpy(even, e.data(), e.size());
    std::memcpy(odd, o.data(), o.size());
    std::memcpy(scales, s.data(), s.size() * sizeof(float));
}

// M>1 activation quantiser, one scale per 32 values, natural k order.
void ref_quantize_a_q8_blocks(const float* a, int m, int k, int lda, int8_t* q,
                              float* scales) {
    std::vector<int8_t> qa;
    std::vector<float> s;
    quantize_a_q8_blocks(a, m, k, lda, k, qa, s);
    std::memcpy(q, qa.data(), qa.size());
    std::memcpy(scales, s.data(), s.size() * sizeof(float));
}

// Row-major int4 bytes [N, K/2] + fp32 scales [N, K/128] -> BG128 blocks.
// `out` must hold ((N+7)/8)*(K/128)*544 bytes.  Returns 0 on success.
int ref_pack_bg128(const uint8_t* rowmajor_q4, const float* scales, int n, int k,
                   uint8_t* out) {
    uint8_t* q4dot = pack_b_q4dot_int4_full(rowmajor_q4, n, k, k);
    if (!q4dot)
        return -1;
    uint8_t* bg = pack_b_q4dot_g128_full(q4dot, scales, n, k, k / 128);
    delete[] q4dot;
    if (!bg)
        return -2;
    std::memcpy(out, bg, pack_b_q4dot_g128_bytes(n, k));
    delete[] bg;
    return 0;
}

// The reference's matmul entry point on a BG128 weight.  On x86 this is the
// W4A32 provider (fp32 activations), not the W4A8 arithmetic.
void ref_matmul_bg128(const float* a, int m, int k, int lda, const void* blocks,
                      int n, float* c, int ldc, int act, int act_n_begin,
                      int act_n_len, int threads) {
    Tensor A = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, k, m, 1, 1,
                              const_cast<float*>(a));
    A.stride[1] = static_cast<size_t>(lda) * sizeof(float);
    Tensor B = make_bg128_weight(blocks, n, k);
    Tensor C = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, n, m, 1, 1, c);
    C.stride[1] = static_cast<size_t>(ldc) * sizeof(float);
    kernel_matmul_fp32(A, B, C, pool_for(threads), static_cast<Activation>(act),
                       act_n_begin, act_n_len);
}

// Average seconds per call of ref_matmul_bg128 over `repeat` calls, rotating
// through `copies` weight buffers laid back to back at `blocks` so a hot cache
// cannot serve the weight stream.
double ref_time_matmul_bg128(const float* a, int m, int k, const void* blocks,
                             size_t copy_stride_bytes, int copies, int n,
                             float* c, int threads, int warmup, int repeat) {
    ThreadPool* pool = pool_for(threads);
    Tensor A = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, k, m, 1, 1,
                              const_cast<float*>(a));
    Tensor C = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, n, m, 1, 1, c);
    auto run = [&](int i) {
        const uint8_t* p = static_cast<const uint8_t*>(blocks) +
                           static_cast<size_t>(i % copies) * copy_stride_bytes;
        Tensor B = make_bg128_weight(p, n, k);
        kernel_matmul_fp32(A, B, C, pool);
    };
    for (int i = 0; i < warmup; ++i)
        run(i);
    auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < repeat; ++i)
        run(warmup + i);
    auto t1 = std::chrono::steady_clock::now();
    return std::chrono::duration<double>(t1 - t0).count() / repeat;
}

int ref_select_moe_routes(const float* logits, int tokens, int num_experts,
                          int top_k, int score_func, int normalize_topk,
                          int32_t* indices, float* weights) {
    mollm::detail::MoeRoutingParams p;
    p.num_experts = num_experts;
    p.top_k = top_k;
    p.score_func = score_func;
    p.normalize_topk = normalize_topk != 0;
    std::vector<int> idx;
    std::vector<float> w;
    if (!mollm::detail::select_moe_routes(logits, tokens, nullptr, p, idx, w))
        return -1;
    for (size_t i = 0; i < idx.size(); ++i)
        indices[i] = idx[i];
    std::memcpy(weights, w.data(), w.size() * sizeof(float));
    return 0;
}

// The same with every routing parameter the reference has (score kind, choice bias, expert
// groups, scaling factor).
int ref_select_moe_routes_ex(const float* logits, int tokens, int num_experts, int top_k,
                             int score_func, int normalize_topk, int num_groups,
                             int topk_groups, float scaling, const float* bias,
                             int32_t* indices, float* weights) {
    mollm::detail::MoeRoutingParams p;
    p.num_experts = num_experts;
    p.top_k = top_k;
    p.score_func = score_func;
    p.normalize_topk = normalize_topk != 0;
    p.num_groups = num_groups;
    p.topk_groups = topk_groups;
    p.scaling_factor = scaling;
    std::vector<int> idx;
    std::vector<float> w;
    if (!mollm::detail::select_moe_routes(logits, tokens, bias, p, idx, w))
        return -1;
    for (size_t i = 0; i < idx.size(); ++i)
        indices[i] = idx[i];
    std::memcpy(weights, w.data(), w.size() * sizeof(float));
    return 0;
}

// Routed MoE op with an fp16 router [E, H], BG128 gate_up [E*2I, H] and BG128
// down [E*H, I] aggregates, softmax top-k routing and no shared expert (the
// Qwen3-MoE configuration, models/qwen3_moe.py:782-797 of the reference).
int ref_moe_bg128(const float* hidden, int tokens, int hidden_size,
                  const uint16_t* router_fp16, int num_experts, int top_k,
                  int intermediate, const void* gate_up_blocks,
                  const void* down_blocks, float* out, int threads) {
    Tensor x = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, hidden_size,
                              tokens, 1, 1, const_cast<float*>(hidden));
    Tensor router = Tensor::create(Precision::FP16, MemoryType::EXTERNAL,
                                   num_experts, hidden_size, 1, 1,
                                   const_cast<uint16_t*>(router_fp16));
    Tensor gu = make_bg128_weight(gate_up_blocks, num_experts * 2 * intermediate,
                                  hidden_size);
    Tensor dn = make_bg128_weight(down_blocks, num_experts * hidden_size,
                                  intermediate);
    Tensor y = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, hidden_size,
                              tokens, 1, 1, out);
    std::vector<const Tensor*> inputs = {&x, &router, &gu, &dn};
    bool ok = kernel_qwen3_moe(inputs, y, pool_for(threads), hidden_size,
                               num_experts, top_k, intermediate, 0,
                               /*router_score_func=*/0, /*norm_topk_prob=*/true,
                               /*has_shared_expert=*/false);
    return ok ? 0 : -1;
}

// Greedy token: the stateless sampling entry at temperature 0 is argmax_token
// (engine/sampler.cpp:31-77, :166-172, :458-462).
int ref_greedy_token(const float* logits, int vocab_size) {
    std::vector<float> copy(logits, logits + (vocab_size > 0 ? vocab_size : 0));
    unsigned int seed = 1;
    return sample_token(copy.data(), vocab_size, 0.0f, 1, 0.0f, &seed);
}

// ---- the operators between a decoder layer's matmuls (rows = tokens, features contiguous)

void ref_rms_norm(const float* x, int rows, int dim, const float* weight, float eps,
                  float* out) {
    Tensor xt = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, dim, rows, 1, 1,
                               const_cast<float*>(x));
    Tensor wt = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, dim, 1, 1, 1,
                               const_cast<float*>(weight));
    Tensor ot = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, dim, rows, 1, 1, out);
    kernel_rms_norm(xt, wt, eps, ot);
}

void ref_add_rms_norm(float* residual, const float* update, int rows, int dim,
                      const float* weight, float eps, float* out) {
    Tensor rt = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, dim, rows, 1, 1, residual);
    Tensor ut = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, dim, rows, 1, 1,
                               const_cast<float*>(update));
    Tensor wt = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, dim, 1, 1, 1,
                               const_cast<float*>(weight));
    Tensor ot = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, dim, rows, 1, 1, out);
    kernel_add_rms_norm(rt, ut, wt, eps, ot, nullptr);
}

void ref_swiglu(const float* merged, int rows, int intermediate, float* out) {
    Tensor mt = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, 2 * intermediate, rows, 1, 1,
                               const_cast<float*>(merged));
    Tensor ot = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, intermediate, rows, 1, 1,
                               out);
    std::vector<const Tensor*> in = {&mt};
    kernel_elementwise(OpType::SWIGLU, in, &ot, nullptr);
}

// x, out: [tokens][heads][dim]; cos, sin: [tokens][rope_dim/2]; halves form (interleave off)
void ref_rope(const float* x, int tokens, int heads, int dim, const float* cosv,
              const float* sinv, int rope_dim, float* out) {
    Tensor xt = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, dim, tokens, heads, 1,
                               const_cast<float*>(x));
    Tensor ot = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, dim, tokens, heads, 1, out);
    for (Tensor* t : {&xt, &ot}) {  // token stride = heads * dim, head stride = dim
        t->stride[1] = sizeof(float) * static_cast<size_t>(heads) * dim;
        t->stride[2] = sizeof(float) * static_cast<size_t>(dim);
    }
    Tensor ct = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, rope_dim / 2, tokens, 1, 1,
                               const_cast<float*>(cosv));
    Tensor st = Tensor::create(Precision::FP32, MemoryType::EXTERNAL, rope_dim / 2, tokens, 1, 1,
                               const_cast<float*>(sinv));
    kernel_rope(xt, ct, st, rope_dim, false, ot);
}

// one head: query [q_tokens][dim], key / value [k_tokens][dim], mask [q_tokens][k_tokens] or null
void ref_sdpa_head(const float* query, const float* key, const float* value, float* output,
                   int query_tokens, int key_tokens, int key_dim, int value_dim, float scale,
                   const float* mask) {
    sdpa_x86_avx512_head(query, key, value, output, query_tokens, key_tokens, key_dim, value_dim,
                         scale, mask);
}

}  // extern "C"


// The reference's engine on a .mollm package, CPU device, greedy sampling: the first token
// after the prompt and steps - 1 more go to tokens_out; last_logits_out (vocab floats, may be
// null) receives the logits of the prompt's last position.  Returns 0, or a negative code.
extern "C" int ref_engine_generate(const char* package_path, const int* prompt, int n_prompt,
                                   int steps, int n_ctx, int threads, int* tokens_out,
                                   float* last_logits_out, int vocab) {
    if (!package_path || !prompt || n_prompt <= 0 || steps <= 0 || !tokens_out)
        return -1;
    LLMEngine engine;
    EngineConfig config;
    config.package_path = package_path;
    config.device = Device::CPU;
    config.n_ctx = n_ctx;
    config.num_threads = threads;
    config.weight_loading = WeightLoadingMode::RESIDENT;
    config.sampling.temperature = 0.0f;
    if (!engine.load(config))
        return -2;
    const std::vector<int> ids(prompt, prompt + n_prompt);
    if (last_logits_out) {
        Tensor hidden = engine.prefill_hidden(ids);
        if (!hidden.data)
            return -3;
        const std::vector<float> logits = engine.run_lmhead_raw(hidden, n_prompt);
        if (static_cast<int>(logits.size()) != vocab)
            return -4;
        std::memcpy(last_logits_out, logits.data(), sizeof(float) * vocab);
        engine.reset();
    }
    int token = engine.prefill(ids);
    if (token < 0)
        return -5;
    tokens_out[0] = token;
    for (int i = 1; i < steps; ++i) {
        token = engine.decode(token);
        if (token < 0)
            return -6;
        tokens_out[i] = token;
    }
    return 0;
}


// ---------------------------------------------------------------------------------------
// The reference's CPU engine with W4A8 matmuls.  On x86 the engine's INT4 matmuls go through
// the provider seam mollm::cpu::matmul_int4_packed (kernels/cpu_platform.h:75-79, x86
// definition kernels/cpu_platform_x86.cpp:128-270: fp32 activations times dequantised
// weights).  The definition below sits in front of the reference library's in symbol
// lookup: switched off it forwards to the reference's own; switched on it answers BG128
// matmuls with the oracle's W4A8 arithmetic under the reference's rule per row count (one
// row: per 128 values, kernels/matmul_w4.cpp:1058-1075; several: per 32, :1125-1154), which is
// what the reference's ARM build computes.  Everything else of a run -- graph executor,
// norms, rotary embedding, attention, MoE control flow, sampler -- stays the reference's code.
extern "C" int orc_matmul_w4(const uint8_t* blocks, int n, int k, const float* x, int m, int lda,
                             float* y, int ldc, int act_rule, int32_t* group_sums);

namespace {
int g_w4a8_provider = 0;
using ProviderFn = bool (*)(const Tensor&, const Tensor&, Tensor&, int, int, ThreadPool*);
}  // namespace

extern "C" void ref_set_w4a8_provider(int on) { g_w4a8_provider = on; }

namespace mollm::cpu {
bool matmul_int4_packed(const Tensor& A, const Tensor& B, Tensor& C, int lda, int ldc,
                        ThreadPool* thread_pool) {
    if (g_w4a8_provider && B.is_q4_g128_packed && B.q4_g128_data && B.group_size == 128 &&
        A.shape[0] % 128 == 0) {
        const int m = static_cast<int>(A.shape[1]);
        const int k = static_cast<int>(A.shape[0]);
        const int n = static_cast<int>(B.shape[0]);
        return orc_matmul_w4(static_cast<const uint8_t*>(B.q4_g128_data), n, k, A.ptr<float>(),
                             m, lda, C.ptr<float>(), ldc, m == 1 ? 128 : 32, nullptr) == 0;
    }
    static ProviderFn next = reinterpret_cast<ProviderFn>(dlsym(
        RTLD_NEXT, "_ZN5mollm3cpu18matmul_int4_packedERK6TensorS3_RS1_iiP10ThreadPool"));
    return next ? next(A, B, C, lda, ldc, thread_pool) : false;
}
}  // namespace mollm::cpu
