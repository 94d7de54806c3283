/* TEST INFRASTRUCTURE ONLY -- never linked into or called by the product path.
 *
 * CPU restatement, in plain C, of the reference's W4G128 / W4A8 arithmetic.
 * The W4A8 kernels of the reference are ARM-NEON only and cannot be executed
 * on an x86 host, so this file restates them scalar-wise with the same
 * rounding points.  Each function cites the reference file:line it follows.
 *
 * How this oracle is pinned (tests/test_oracle_pins.py, tests/golden/):
 *   - activation quantisers: bit-exact against the reference's own portable
 *     quantize_a_q8_g128_even_odd / quantize_a_q8_blocks, which do run on x86;
 *   - BG128 block layout: byte-exact against the reference's packers;
 *   - block decode + group structure: the exact dequantised product in fp64
 *     against the reference's x86 W4A32 kernel_matmul_fp32 (tolerance 1e-5
 *     relative L2) on the reference's own closed-form test inputs;
 *   - routing: bit-exact indices, weights to 1 ulp, against select_moe_routes;
 *   - MoE control flow: W4A32 expert mode against kernel_qwen3_moe (1e-5).
 * What no reference test or runnable reference code pins: the int32 group
 * accumulators and the W4A8 fp32 chain of the NEON kernels.  Those are pinned
 * only by composition of the pinned pieces plus the restated loop below.
 */
#ifndef W4A8_ORACLE_H
#define W4A8_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_BG128_BLOCK_BYTES = 544 };

/* activation-quantisation rules */
enum {
    ORC_ACT_G128 = 128, /* one scale per 128 values (reference M==1 rule)   */
    ORC_ACT_G32 = 32,   /* one scale per 32 values  (reference M>1 rule)    */
    ORC_ACT_G32_I8MM = 33, /* the same rule as ARM CPUs with int8 matrix
                              instructions associate it (matmul only)        */
    ORC_ACT_F64 = 0     /* no activation quantisation: exact fp64 product   */
};

/* 0: exp through the host libm's expf, as the reference built here does (default);
 * 1: exp evaluated in double and rounded once (what the GPU kernels do). */
void orc_set_exp_mode(int correctly_rounded);

size_t orc_bg128_bytes(int n, int k);
void orc_bg128_encode(const int8_t* q, const float* scales, int n, int k,
                      uint8_t* blocks);
void orc_bg128_decode(const uint8_t* blocks, int n, int k, int8_t* q,
                      float* scales);

void orc_quantize_a_g128(const float* x, int k, int8_t* q, float* scales);
void orc_quantize_a_g128_even_odd(const float* x, int k, int8_t* even,
                                  int8_t* odd, float* scales);
void orc_quantize_a_g32(const float* x, int m, int k, int lda, int8_t* q,
                        float* scales);

void orc_group_sums_g128(const uint8_t* blocks, int n, int k, const int8_t* qa,
                         int32_t* sums);

/* y[m][n] for one activation rule; group_sums may be NULL, else receives the
 * int32 accumulators [m][n][k/128] (ORC_ACT_G128) or [m][n][k/32] (ORC_ACT_G32). */
int orc_matmul_w4(const uint8_t* blocks, int n, int k, const float* x, int m,
                  int lda, float* y, int ldc, int act_rule, int32_t* group_sums);

void orc_apply_activation(float* y, int m, int n, int ldc, int act,
                          int act_n_begin, int act_n_len);

int orc_moe_select_routes_softmax(const float* logits, int tokens,
                                  int num_experts, int top_k, int32_t* indices,
                                  float* weights);

void orc_router_logits(const float* hidden, int tokens, int hidden_size, int ldx,
                       const uint16_t* router_fp16, int num_experts,
                       float* logits);

/* expert_rule: ORC_ACT_G128 (every routed row uses the per-128 rule),
 * ORC_ACT_G32 (the reference's own switch: an expert holding exactly one row
 * uses per-128, more than one row per-32), ORC_ACT_F64 (exact W4A32 product).
 * Optional outputs (may be NULL): logits [tokens][E], indices/weights
 * [tokens][top_k]. */
int orc_moe_forward(const float* hidden, int tokens, int hidden_size, int ldx,
                    const uint16_t* router_fp16, int num_experts, int top_k,
                    int intermediate, const uint8_t* gate_up_blocks,
                    const uint8_t* down_blocks, float* out, int ldo,
                    int expert_rule, float* logits_out, int32_t* indices_out,
                    float* weights_out);

/* The combine step of kernel_qwen3_moe alone (kernels/moe.cpp:642-645, :966,
 * :1100-1110): out[t] starts at 0 and takes fmaf(w, y, out[t]) for the token's
 * routes in ascending expert id (the order the expert loop visits them).
 * route_out fp32 [tokens*top_k][H], row t*top_k+j = the j-th route's expert
 * output.  Used to check the expert-parallel split of the op. */
void orc_moe_combine(const float* route_out, int tokens, int hidden_size, int top_k,
                     const int32_t* indices, const float* weights, float* out, int ldo);

/* Greedy token of one row of logits (engine/sampler.cpp:72-77, the scalar form
 * of argmax_token): best = 0; every i with logits[i] > logits[best] takes over.
 * The first maximum wins; a NaN never wins, except at index 0 where nothing
 * beats it.  vocab_size <= 0 gives 0 (engine/sampler.cpp:169-170). */
int orc_argmax_token(const float* logits, int vocab_size);

float orc_fp16_to_fp32(uint16_t h);

#ifdef __cplusplus
}
#endif
/* The operators between a decoder layer's matmuls, from the reference's x86 build (rows =
 * tokens, features contiguous): kernels/norm.cpp:13-31, :123-190; kernels/elementwise.cpp:
 * 565-569; kernels/rope.cpp:11-50; kernels/attention_x86_avx512.cpp:12-109. */
void orc_rms_norm(const float* x, int rows, int dim, const float* weight, float eps,
                  float* out);
void orc_add_rms_norm(float* residual, const float* update, int rows, int dim,
                      const float* weight, float eps, float* out);
void orc_swiglu(const float* merged, int rows, int intermediate, float* out);
void orc_rope(const float* x, int tokens, int heads, int dim, const float* cosv,
              const float* sinv, int rope_dim, float* out);
void orc_sdpa_head(const float* query, const float* key, const float* value, float* output,
                   int query_tokens, int key_tokens, int key_dim, int value_dim, float scale,
                   const float* mask);

/* Which build of the reference the MoE operator's two order-sensitive sums follow: 0 (default)
 * the ARM reading the GPU implements, 1 the x86 AVX-512 build (for bit-for-bit comparison with
 * the engine compiled on an x86 host). */
void orc_set_moe_host_build(int x86_avx512);

/* Routing with the reference's other score kinds (1 logistic, 2 sqrt(softplus)), optional
 * choice bias, expert groups, optional normalisation and a scaling factor
 * (kernels/moe_routing.cpp:25-169); kind 0 forwards to the softmax form above. */
int orc_moe_select_routes(const float* logits, int tokens, int num_experts, int top_k,
                          int score_kind, int normalize, int groups, int topk_groups,
                          float scaling, const float* bias, int32_t* indices, float* weights);

/* Rotary tables as the reference's engine fills them (engine/input_prep.cpp:18-31). */
void orc_rope_tables(float* cos_out, float* sin_out, int positions, int first_position,
                     int rope_dim, float rope_theta);

#endif
