/* TEST INFRASTRUCTURE ONLY -- see w4a8_oracle.h for scope and pinning.
 *
 * Compile with -ffp-contract=off: the only fused multiply-adds are the
 * explicit fmaf() calls that mirror the reference's vfmaq_f32.
 */
#include "w4a8_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* exp of a float.  The reference calls std::exp on a float (kernels/activations.h:76-99,
 * kernels/moe_routing.cpp:157-166, kernels/moe.cpp:160-183), i.e. the platform libm's expf,
 * which is within one ulp of the correctly rounded value but not always equal to it (glibc:
 * about 6 in 10000 arguments differ in the last bit).  Mode 0 (default) calls expf, like the
 * reference built on this host; mode 1 evaluates in double and rounds once, which is what
 * the GPU kernels do and is independent of the host's libm. */
static int g_exp_mode = 0;
void orc_set_exp_mode(int correctly_rounded) { g_exp_mode = correctly_rounded != 0; }
static float orc_exp(float x) { return g_exp_mode ? (float)exp((double)x) : expf(x); }

/* ---------------------------------------------------------------- fp16 -- */

float orc_fp16_to_fp32(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) << 31;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ff;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* ------------------------------------------------------ BG128 blocks (a1) --
 * Layout authority: kernels/quant_layouts.h:9-14 (struct), packer
 * kernels/matmul_pack.cpp:641-688, element addressing kernels/moe.cpp:110-120.
 * Block (n8, g) sits at index n8*(K/128)+g; bytes 0..31 are eight fp32 row
 * scales; byte 32 + ((sub*8 + row)*16) + j holds k = g*128 + sub*32 + 2j in
 * its low nibble and k+1 in its high nibble, two's-complement 4-bit.         */

size_t orc_bg128_bytes(int n, int k) {
    return (size_t)((n + 7) / 8) * (size_t)(k / 128) * ORC_BG128_BLOCK_BYTES;
}

static inline const uint8_t* block_at(const uint8_t* blocks, int k, int row,
                                      int g) {
    return blocks +
           ((size_t)(row / 8) * (size_t)(k / 128) + (size_t)g) * ORC_BG128_BLOCK_BYTES;
}

static inline int nibble_value(const uint8_t* blk, int row, int kk) {
    /* kk = position inside the 128-wide group */
    uint8_t byte = blk[32 + (((kk >> 5) * 8 + (row & 7)) * 16) + ((kk & 31) >> 1)];
    int v = (kk & 1) ? (byte >> 4) : (byte & 15);
    return v >= 8 ? v - 16 : v; /* kernels/matmul_w4.cpp:8-13 */
}

static inline float block_scale(const uint8_t* blk, int row) {
    float s;
    memcpy(&s, blk + 4 * (row & 7), 4);
    return s;
}

void orc_bg128_encode(const int8_t* q, const float* scales, int n, int k,
                      uint8_t* blocks) {
    int groups = k / 128;
    memset(blocks, 0, orc_bg128_bytes(n, k));
    for (int row = 0; row < n; ++row) {
        for (int g = 0; g < groups; ++g) {
            uint8_t* blk = (uint8_t*)block_at(blocks, k, row, g);
            memcpy(blk + 4 * (row & 7), &scales[(size_t)row * groups + g], 4);
            for (int kk = 0; kk < 128; ++kk) {
                uint8_t nib = (uint8_t)q[(size_t)row * k + g * 128 + kk] & 15;
                uint8_t* byte =
                    blk + 32 + (((kk >> 5) * 8 + (row & 7)) * 16) + ((kk & 31) >> 1);
                *byte |= (kk & 1) ? (uint8_t)(nib << 4) : nib;
            }
        }
    }
}

void orc_bg128_decode(const uint8_t* blocks, int n, int k, int8_t* q,
                      float* scales) {
    int groups = k / 128;
    for (int row = 0; row < n; ++row) {
        for (int g = 0; g < groups; ++g) {
            const uint8_t* blk = block_at(blocks, k, row, g);
            scales[(size_t)row * groups + g] = block_scale(blk, row);
            for (int kk = 0; kk < 128; ++kk)
                q[(size_t)row * k + g * 128 + kk] = (int8_t)nibble_value(blk, row, kk);
        }
    }
}

/* ------------------------------------------- activation quantisers (a2, a5) --
 * kernels/matmul_quant.cpp:578-641 (per 128, M==1) and :280-329 (per 32, M>1):
 * amax over the group; scale = amax>0 ? amax/127 : 1; inv = amax>0 ? 127/amax
 * : 0; q = clamp(nearbyint(x*inv), -127, 127) with round-to-nearest-even.   */

static void quantize_group(const float* x, int len, int8_t* q, float* scale) {
    float amax = 0.f;
    for (int i = 0; i < len; ++i) {
        float a = fabsf(x[i]);
        if (a > amax)
            amax = a;
    }
    float s = (amax > 0.f) ? (amax / 127.f) : 1.f;
    float inv = (amax > 0.f) ? (127.f / amax) : 0.f;
    *scale = s;
    for (int i = 0; i < len; ++i) {
        float scaled = x[i] * inv;
        int v = (int)nearbyintf(scaled);
        if (v > 127)
            v = 127;
        if (v < -127)
            v = -127;
        q[i] = (int8_t)v;
    }
}

void orc_quantize_a_g128(const float* x, int k, int8_t* q, float* scales) {
    for (int g = 0; g < k / 128; ++g)
        quantize_group(x + (size_t)g * 128, 128, q + (size_t)g * 128, &scales[g]);
}

void orc_quantize_a_g128_even_odd(const float* x, int k, int8_t* even,
                                  int8_t* odd, float* scales) {
    int8_t* q = (int8_t*)malloc((size_t)k);
    orc_quantize_a_g128(x, k, q, scales);
    for (int qb = 0; qb < k / 32; ++qb) {
        for (int i = 0; i < 16; ++i) {
            even[qb * 16 + i] = q[qb * 32 + 2 * i];
            odd[qb * 16 + i] = q[qb * 32 + 2 * i + 1];
        }
    }
    free(q);
}

void orc_quantize_a_g32(const float* x, int m, int k, int lda, int8_t* q,
                        float* scales) {
    int blocks = k / 32;
    for (int r = 0; r < m; ++r)
        for (int qb = 0; qb < blocks; ++qb)
            quantize_group(x + (size_t)r * lda + qb * 32, 32,
                           q + (size_t)r * k + qb * 32,
                           &scales[(size_t)r * blocks + qb]);
}

/* ----------------------------------------------- integer dot products (a3) --
 * kernels/matmul_w4.cpp:16-45: the NEON kernel multiplies the nibble, left-
 * aligned in its byte (i.e. 16*q4), with the int8 activation and accumulates
 * in int32; kernels/matmul_w4.cpp:52-58 divides by 16 on conversion.  The sum
 * of 16*q4*q8 over a group is an exact multiple of 16, so the value converted
 * to float equals the plain sum of q4*q8 computed here.                      */

static int32_t dot_span(const uint8_t* blk, int row, int kk0, int len,
                        const int8_t* qa) {
    int32_t acc = 0;
    for (int i = 0; i < len; ++i)
        acc += nibble_value(blk, row, kk0 + i) * (int32_t)qa[i];
    return acc;
}

void orc_group_sums_g128(const uint8_t* blocks, int n, int k, const int8_t* qa,
                         int32_t* sums) {
    int groups = k / 128;
    for (int row = 0; row < n; ++row)
        for (int g = 0; g < groups; ++g)
            sums[(size_t)row * groups + g] =
                dot_span(block_at(blocks, k, row, g), row, 0, 128, qa + g * 128);
}

/* --------------------------------------------------------- matmul (a3, a6) --
 * ORC_ACT_G128, row by row: kernels/matmul_w4.cpp:211-295 -- per group,
 *     acc = fma(float(dot128), fp32(bscale * ascale[g]), acc), g ascending.
 * ORC_ACT_G32: kernels/matmul_w4.cpp:785-901 (dot-product variant) -- per
 *     32-block qb, acc = fma(float(dot32), fp32(bscale[g] * ascale[m][qb]), acc).
 * ORC_ACT_G32_I8MM: the same per-32 quantisation as the reference computes it on ARM CPUs
 *     that have the int8 matrix instructions (kernels/matmul_w4.cpp:1018-1030, 1160-1167 ->
 *     kernels/matmul_w4_i8mm.cpp:129-207): per group, the four blocks are first summed with
 *     their activation scales, t = fma(float(dot32_b), ascale[m][b], t) for b = 0..3 from
 *     t = 0 (:100-121, the scvtf #4 undoes the factor 16 of the left-aligned nibbles), then
 *     acc = fma(t, bscale[g], acc) (:172-179) -- another association of the same products,
 *     so the two ARM paths agree to fp32 rounding, not bit for bit.  The GPU kernels
 *     implement ORC_ACT_G32 (the dot-product path, which every ARMv8.2 CPU runs).
 * ORC_ACT_F64: exact dequantised product, the yardstick the reference's x86
 *     W4A32 kernels (kernels/matmul_x86_avx512.cpp:112-213) approximate.      */

static int32_t dot_i8(const int8_t* a, const int8_t* b, int len) {
    int32_t acc = 0;
    for (int i = 0; i < len; ++i)
        acc += (int32_t)a[i] * (int32_t)b[i];
    return acc;
}

int orc_matmul_w4(const uint8_t* blocks, int n, int k, const float* x, int m,
                  int lda, float* y, int ldc, int act_rule, int32_t* group_sums) {
    if (k <= 0 || k % 128 != 0 || n <= 0 || m <= 0)
        return -1;
    if (act_rule != ORC_ACT_G128 && act_rule != ORC_ACT_G32 &&
        act_rule != ORC_ACT_G32_I8MM && act_rule != ORC_ACT_F64)
        return -2;
    int groups = k / 128;
    int qblocks = k / 32;
    /* decode the blocks once (a1); the arithmetic below is per element */
    int8_t* wq = (int8_t*)malloc((size_t)n * k);
    float* ws = (float*)malloc(sizeof(float) * (size_t)n * groups);
    int8_t* qa = (int8_t*)malloc((size_t)k);
    float* as = (float*)malloc(sizeof(float) * (size_t)qblocks);
    orc_bg128_decode(blocks, n, k, wq, ws);
    for (int r = 0; r < m; ++r) {
        const float* xr = x + (size_t)r * lda;
        float* yr = y + (size_t)r * ldc;
        if (act_rule == ORC_ACT_G128) {
            orc_quantize_a_g128(xr, k, qa, as);
            for (int row = 0; row < n; ++row) {
                float acc = 0.f;
                for (int g = 0; g < groups; ++g) {
                    int32_t d = dot_i8(wq + (size_t)row * k + g * 128, qa + g * 128, 128);
                    if (group_sums)
                        group_sums[((size_t)r * n + row) * groups + g] = d;
                    float sc = ws[(size_t)row * groups + g] * as[g];
                    acc = fmaf((float)d, sc, acc);
                }
                yr[row] = acc;
            }
        } else if (act_rule == ORC_ACT_G32) {
            orc_quantize_a_g32(xr, 1, k, k, qa, as);
            for (int row = 0; row < n; ++row) {
                float acc = 0.f;
                for (int qb = 0; qb < qblocks; ++qb) {
                    int32_t d = dot_i8(wq + (size_t)row * k + qb * 32, qa + qb * 32, 32);
                    if (group_sums)
                        group_sums[((size_t)r * n + row) * qblocks + qb] = d;
                    float sc = ws[(size_t)row * groups + qb / 4] * as[qb];
                    acc = fmaf((float)d, sc, acc);
                }
                yr[row] = acc;
            }
        } else if (act_rule == ORC_ACT_G32_I8MM) {
            orc_quantize_a_g32(xr, 1, k, k, qa, as);
            for (int row = 0; row < n; ++row) {
                float acc = 0.f;
                for (int g = 0; g < groups; ++g) {
                    float t = 0.f;
                    for (int b = 0; b < 4; ++b) {
                        int qb = g * 4 + b;
                        int32_t d = dot_i8(wq + (size_t)row * k + qb * 32, qa + qb * 32, 32);
                        if (group_sums)
                            group_sums[((size_t)r * n + row) * qblocks + qb] = d;
                        t = fmaf((float)d, as[qb], t);
                    }
                    acc = fmaf(t, ws[(size_t)row * groups + g], acc);
                }
                yr[row] = acc;
            }
        } else {
            for (int row = 0; row < n; ++row) {
                double acc = 0.0;
                for (int g = 0; g < groups; ++g) {
                    double part = 0.0;
                    for (int kk = 0; kk < 128; ++kk)
                        part += (double)wq[(size_t)row * k + g * 128 + kk] *
                                (double)xr[g * 128 + kk];
                    acc += part * (double)ws[(size_t)row * groups + g];
                }
                yr[row] = (float)acc;
            }
        }
    }
    free(wq);
    free(ws);
    free(qa);
    free(as);
    return 0;
}

/* ------------------------------------------------- fused activation (a7) --
 * kernels/matmul_internal.h:73-119 (column range) and kernels/activations.h:
 * 76-99 (scalar forms): applied after the matmul on columns
 * [act_n_begin, act_n_begin+act_n_len); act_n_len < 0 means every column.    */

static float activation_scalar(float v, int act) {
    switch (act) {
    case 1: { /* SILU */
        float s = 1.f / (1.f + orc_exp(-v));
        return v * s;
    }
    case 2: { /* GELU, tanh form */
        const float c = 0.7978845608f;
        float v3 = v * v * v;
        float inner = c * (v + 0.044715f * v3);
        return 0.5f * v * (1.f + tanhf(inner));
    }
    case 3:
        return v > 0.f ? v : 0.f;
    case 4: {
        float r = v > 0.f ? v : 0.f;
        return r * r;
    }
    default:
        return v;
    }
}

void orc_apply_activation(float* y, int m, int n, int ldc, int act,
                          int act_n_begin, int act_n_len) {
    if (act == 0 || act_n_len == 0)
        return;
    int full = act_n_len < 0 || (act_n_begin == 0 && act_n_len >= n);
    int begin = full ? 0 : act_n_begin;
    int end = full ? n : act_n_begin + act_n_len;
    if (end > n)
        end = n;
    for (int r = 0; r < m; ++r)
        for (int c = begin; c < end; ++c)
            y[(size_t)r * ldc + c] = activation_scalar(y[(size_t)r * ldc + c], act);
}

/* -------------------------------------------------------- routing (a10) --
 * kernels/moe_routing.cpp:129-142 (insertion top-k with strict '>', so equal
 * logits keep the lower expert id first) and :157-166 (softmax over the k
 * selected logits, max-subtracted; the first selected logit is the max).     */

int orc_moe_select_routes_softmax(const float* logits, int tokens,
                                  int num_experts, int top_k, int32_t* indices,
                                  float* weights) {
    if (!logits || tokens <= 0 || num_experts <= 0 || top_k <= 0 ||
        top_k > num_experts)
        return -1;
    for (int t = 0; t < tokens; ++t) {
        const float* row = logits + (size_t)t * num_experts;
        int32_t* idx = indices + (size_t)t * top_k;
        float* w = weights + (size_t)t * top_k;
        for (int j = 0; j < top_k; ++j) {
            idx[j] = 0;
            w[j] = -INFINITY;
        }
        for (int e = 0; e < num_experts; ++e) {
            float v = row[e];
            for (int j = 0; j < top_k; ++j) {
                if (v > w[j]) {
                    for (int s = top_k - 1; s > j; --s) {
                        w[s] = w[s - 1];
                        idx[s] = idx[s - 1];
                    }
                    w[j] = v;
                    idx[j] = e;
                    break;
                }
            }
        }
        float maximum = w[0];
        float sum = 0.f;
        for (int j = 0; j < top_k; ++j) {
            w[j] = orc_exp(w[j] - maximum);
            sum += w[j];
        }
        float inverse = sum > 0.f ? 1.f / sum : 0.f;
        for (int j = 0; j < top_k; ++j)
            w[j] *= inverse;
    }
    return 0;
}

/* Router logits (kernels/moe.cpp:650-658): hidden[tokens,H] x router[E,H]^T
 * with an fp16, unquantised router weight.  The reference leaves the fp32
 * summation order to whichever dense kernel the host selects; the oracle
 * accumulates in fp64 and rounds once, the order-free reading of that sum.  */
/* Two places of the MoE operator are summed in an order that depends on how the reference
 * was built.  Mode 0 (default, what the GPU follows): router logits as the exact dot product
 * rounded once, the weighted sum of expert outputs with one fused multiply-add per term (the
 * ARM build contracts `dst += w * src`, kernels/moe.cpp:1100-1110).  Mode 1, the x86 AVX-512
 * build as compiled here: router logits through its fp16 dense kernel
 * (kernels/matmul_x86_avx512.cpp:76-110: two 16-lane fused accumulators over alternate
 * 16-feature chunks, added lane-wise, a last 16-chunk into the sum, the 16 lanes reduced by
 * halves, a scalar tail), and `w * src` rounded before the addition (no fused instruction in
 * that translation unit).  Mode 1 exists so that the whole operator can be compared bit for
 * bit with the x86 engine.                                                                   */
static int g_moe_host_build = 0;

void orc_set_moe_host_build(int x86_avx512) { g_moe_host_build = x86_avx512 ? 1 : 0; }

static float router_dot_x86_avx512(const float* a, const uint16_t* b_fp16, int count) {
    float first[16] = {0}, second[16] = {0}, v[16];
    int i = 0;
    for (; i + 31 < count; i += 32)
        for (int l = 0; l < 16; ++l) {
            first[l] = fmaf(a[i + l], orc_fp16_to_fp32(b_fp16[i + l]), first[l]);
            second[l] = fmaf(a[i + 16 + l], orc_fp16_to_fp32(b_fp16[i + 16 + l]), second[l]);
        }
    for (int l = 0; l < 16; ++l)
        v[l] = first[l] + second[l];
    for (; i + 15 < count; i += 16)
        for (int l = 0; l < 16; ++l)
            v[l] = fmaf(a[i + l], orc_fp16_to_fp32(b_fp16[i + l]), v[l]);
    for (int width = 8; width >= 1; width >>= 1)
        for (int l = 0; l < width; ++l)
            v[l] = v[l] + v[l + width];
    float sum = v[0];
    for (; i < count; ++i)
        sum += a[i] * orc_fp16_to_fp32(b_fp16[i]);
    return sum;
}

void orc_router_logits(const float* hidden, int tokens, int hidden_size, int ldx,
                       const uint16_t* router_fp16, int num_experts,
                       float* logits) {
    for (int t = 0; t < tokens; ++t)
        for (int e = 0; e < num_experts; ++e) {
            if (g_moe_host_build) {
                logits[(size_t)t * num_experts + e] = router_dot_x86_avx512(
                    hidden + (size_t)t * ldx, router_fp16 + (size_t)e * hidden_size,
                    hidden_size);
                continue;
            }
            double acc = 0.0;
            for (int d = 0; d < hidden_size; ++d)
                acc += (double)hidden[(size_t)t * ldx + d] *
                       (double)orc_fp16_to_fp32(router_fp16[(size_t)e * hidden_size + d]);
            logits[(size_t)t * num_experts + e] = (float)acc;
        }
}

/* ------------------------------------------------------------ MoE (a11) --
 * kernels/moe.cpp:576-1129: zero the output (:642-645); router logits; routes;
 * counting-sort compaction, tokens ascending inside each expert (:759-776);
 * experts in ascending id (:966): gather, gate_up [2I,H] matmul, silu(gate)*up
 * with gate = rows [0,I) and up = rows [I,2I) (:160-183, :1065-1069), down
 * [H,I] matmul, out[t] += w * y (:1100-1110).  Expert e owns rows e*2I.. of
 * gate_up and e*H.. of down (:1022-1027), both multiples of 8 rows (:319-328). */

int orc_moe_forward(const float* hidden, int tokens, int hidden_size, int ldx,
                    const uint16_t* router_fp16, int num_experts, int top_k,
                    int intermediate, const uint8_t* gate_up_blocks,
                    const uint8_t* down_blocks, float* out, int ldo,
                    int expert_rule, float* logits_out, int32_t* indices_out,
                    float* weights_out) {
    if (hidden_size % 128 || intermediate % 128 || (2 * intermediate) % 8 ||
        hidden_size % 8)
        return -1;
    size_t tk = (size_t)tokens * top_k;
    float* logits = (float*)malloc(sizeof(float) * (size_t)tokens * num_experts);
    int32_t* idx = (int32_t*)malloc(sizeof(int32_t) * tk);
    float* wts = (float*)malloc(sizeof(float) * tk);
    int* counts = (int*)calloc((size_t)num_experts + 1, sizeof(int));
    int* offsets = (int*)calloc((size_t)num_experts + 1, sizeof(int));
    int* cursor = (int*)calloc((size_t)num_experts + 1, sizeof(int));
    int* route_tokens = (int*)malloc(sizeof(int) * tk);
    float* route_weights = (float*)malloc(sizeof(float) * tk);

    for (int t = 0; t < tokens; ++t)
        memset(out + (size_t)t * ldo, 0, sizeof(float) * (size_t)hidden_size);

    orc_router_logits(hidden, tokens, hidden_size, ldx, router_fp16, num_experts,
                      logits);
    int rc = orc_moe_select_routes_softmax(logits, tokens, num_experts, top_k, idx,
                                           wts);
    if (rc == 0) {
        for (size_t i = 0; i < tk; ++i)
            counts[idx[i]]++;
        for (int e = 0; e < num_experts; ++e)
            offsets[e + 1] = offsets[e] + counts[e];
        memcpy(cursor, offsets, sizeof(int) * ((size_t)num_experts + 1));
        for (int t = 0; t < tokens; ++t)
            for (int j = 0; j < top_k; ++j) {
                int e = idx[(size_t)t * top_k + j];
                int pos = cursor[e]++;
                route_tokens[pos] = t;
                route_weights[pos] = wts[(size_t)t * top_k + j];
            }

        int max_count = 0;
        for (int e = 0; e < num_experts; ++e)
            if (counts[e] > max_count)
                max_count = counts[e];
        size_t mc = (size_t)(max_count > 0 ? max_count : 1);
        float* ex = (float*)malloc(sizeof(float) * mc * hidden_size);
        float* gu = (float*)malloc(sizeof(float) * mc * 2 * intermediate);
        float* inter = (float*)malloc(sizeof(float) * mc * intermediate);
        float* dn = (float*)malloc(sizeof(float) * mc * hidden_size);
        size_t gu_expert_bytes = orc_bg128_bytes(2 * intermediate, hidden_size);
        size_t dn_expert_bytes = orc_bg128_bytes(hidden_size, intermediate);

        for (int e = 0; e < num_experts && rc == 0; ++e) {
            int count = counts[e];
            if (count == 0)
                continue;
            int begin = offsets[e];
            for (int i = 0; i < count; ++i)
                memcpy(ex + (size_t)i * hidden_size,
                       hidden + (size_t)route_tokens[begin + i] * ldx,
                       sizeof(float) * (size_t)hidden_size);
            int rule = expert_rule;
            if (expert_rule == ORC_ACT_G32 && count == 1)
                rule = ORC_ACT_G128; /* kernels/matmul_w4.cpp:1058 vs :1125 */
            rc |= orc_matmul_w4(gate_up_blocks + (size_t)e * gu_expert_bytes,
                                2 * intermediate, hidden_size, ex, count,
                                hidden_size, gu, 2 * intermediate, rule, NULL);
            for (int i = 0; i < count; ++i)
                for (int c = 0; c < intermediate; ++c) {
                    float g = gu[(size_t)i * 2 * intermediate + c];
                    float u = gu[(size_t)i * 2 * intermediate + intermediate + c];
                    float s = 1.f / (1.f + orc_exp(-g));
                    inter[(size_t)i * intermediate + c] = (g * s) * u;
                }
            rc |= orc_matmul_w4(down_blocks + (size_t)e * dn_expert_bytes,
                                hidden_size, intermediate, inter, count,
                                intermediate, dn, hidden_size, rule, NULL);
            for (int i = 0; i < count; ++i) {
                float* dst = out + (size_t)route_tokens[begin + i] * ldo;
                const float* src = dn + (size_t)i * hidden_size;
                float w = route_weights[begin + i];
                for (int d = 0; d < hidden_size; ++d) {
                    if (g_moe_host_build) {
                        volatile float product = w * src[d]; /* rounded before the addition */
                        dst[d] = dst[d] + product;
                    } else {
                        dst[d] = fmaf(w, src[d], dst[d]);
                    }
                }
            }
        }
        free(ex);
        free(gu);
        free(inter);
        free(dn);
    }
    if (logits_out)
        memcpy(logits_out, logits, sizeof(float) * (size_t)tokens * num_experts);
    if (indices_out)
        memcpy(indices_out, idx, sizeof(int32_t) * tk);
    if (weights_out)
        memcpy(weights_out, wts, sizeof(float) * tk);
    free(logits);
    free(idx);
    free(wts);
    free(counts);
    free(offsets);
    free(cursor);
    free(route_tokens);
    free(route_weights);
    return rc;
}

void orc_moe_combine(const float* route_out, int tokens, int hidden_size, int top_k,
                     const int32_t* indices, const float* weights, float* out, int ldo) {
    for (int t = 0; t < tokens; ++t) {
        float* dst = out + (size_t)t * ldo;
        const int32_t* idx = indices + (size_t)t * top_k;
        memset(dst, 0, sizeof(float) * (size_t)hidden_size);
        /* visit the routes by ascending expert id; a token's experts are distinct */
        int last = -1;
        for (int step = 0; step < top_k; ++step) {
            int best = -1;
            for (int j = 0; j < top_k; ++j)
                if (idx[j] > last && (best < 0 || idx[j] < idx[best]))
                    best = j;
            if (best < 0)
                break;
            last = idx[best];
            const float* src = route_out + ((size_t)t * top_k + best) * hidden_size;
            float w = weights[(size_t)t * top_k + best];
            for (int d = 0; d < hidden_size; ++d)
                dst[d] = fmaf(w, src[d], dst[d]);
        }
    }
}

/* engine/sampler.cpp:72-77 (and :169-170 for the empty row) */
int orc_argmax_token(const float* logits, int vocab_size) {
    int best = 0;
    for (int i = 1; i < vocab_size; ++i)
        if (logits[i] > logits[best])
            best = i;
    return best;
}


/* ---- the operators between a decoder layer's matmuls --------------------------------
 * Restated from the reference's x86 build (scalar paths unless noted); rows = tokens,
 * features contiguous. */

/* kernel_rms_norm -> rms_norm_scalar (kernels/norm.cpp:13-31): sequential sum of squares. */
void orc_rms_norm(const float* x, int rows, int dim, const float* weight, float eps,
                  float* out) {
    for (int n = 0; n < rows; ++n) {
        const float* xr = x + (size_t)n * dim;
        float* o = out + (size_t)n * dim;
        float sum_sq = 0.f;
        for (int d = 0; d < dim; ++d) {
            float v = xr[d];
            sum_sq += v * v;
        }
        float rms = 1.f / sqrtf(sum_sq / dim + eps);
        for (int d = 0; d < dim; ++d)
            o[d] = xr[d] * rms * weight[d];
    }
}

/* kernel_add_rms_norm (kernels/norm.cpp:123-190), scalar tail: the sum is written back. */
void orc_add_rms_norm(float* residual, const float* update, int rows, int dim,
                      const float* weight, float eps, float* out) {
    for (int n = 0; n < rows; ++n) {
        float* r = residual + (size_t)n * dim;
        const float* u = update + (size_t)n * dim;
        float* o = out + (size_t)n * dim;
        float sum_sq = 0.f;
        for (int d = 0; d < dim; ++d) {
            float value = r[d] + u[d];
            r[d] = value;
            sum_sq += value * value;
        }
        float scale = 1.0f / sqrtf(sum_sq / (float)dim + eps);
        for (int d = 0; d < dim; ++d)
            o[d] = r[d] * scale * weight[d];
    }
}

/* OpType::SWIGLU (kernels/elementwise.cpp:565-569): (g / (1 + exp(-g))) * up. */
void orc_swiglu(const float* merged, int rows, int intermediate, float* out) {
    for (int n = 0; n < rows; ++n) {
        const float* gate = merged + (size_t)n * 2 * intermediate;
        const float* up = gate + intermediate;
        for (int i = 0; i < intermediate; ++i) {
            float g = gate[i];
            out[(size_t)n * intermediate + i] = (g / (1.f + orc_exp(-g))) * up[i];
        }
    }
}

/* kernel_rope -> rope_scalar, halves form (kernels/rope.cpp:11-50).  x, out:
 * [tokens][heads][dim]; cos, sin: [tokens][rope_dim/2]. */
void orc_rope(const float* x, int tokens, int heads, int dim, const float* cosv,
              const float* sinv, int rope_dim, float* out) {
    int half = rope_dim / 2;
    for (int t = 0; t < tokens; ++t)
        for (int h = 0; h < heads; ++h) {
            const float* xr = x + ((size_t)t * heads + h) * dim;
            float* o = out + ((size_t)t * heads + h) * dim;
            for (int d = rope_dim; d < dim; ++d)
                o[d] = xr[d];
            for (int i = 0; i < half; ++i) {
                float x0 = xr[i], x1 = xr[i + half];
                float c = cosv[(size_t)t * half + i], s = sinv[(size_t)t * half + i];
                o[i] = x0 * c - x1 * s;
                o[i + half] = x0 * s + x1 * c;
            }
        }
}

/* sdpa_x86_avx512_head (kernels/attention_x86_avx512.cpp:12-109).  The dot product keeps two
 * 16-lane fused accumulators (lanes i and i + 16 of every 32 features), adds them lane-wise
 * and reduces the 16 lanes the way _mm512_reduce_add_ps expands: halves of 8, of 4, of 2,
 * of 1.  Softmax: max, exp(v - max), sequential sum, times 1 / sum.  P * V: one fused
 * multiply-add per key and feature, keys ascending, zero probabilities skipped. */
static float orc_dot_avx512(const float* a, const float* b, int count) {
    float first[16] = {0}, second[16] = {0};
    int i = 0;
    for (; i + 31 < count; i += 32)
        for (int l = 0; l < 16; ++l) {
            first[l] = fmaf(a[i + l], b[i + l], first[l]);
            second[l] = fmaf(a[i + 16 + l], b[i + 16 + l], second[l]);
        }
    for (; i + 15 < count; i += 16)
        for (int l = 0; l < 16; ++l)
            first[l] = fmaf(a[i + l], b[i + l], first[l]);
    float v[16];
    for (int l = 0; l < 16; ++l)
        v[l] = first[l] + second[l];
    for (int width = 8; width >= 1; width >>= 1)
        for (int l = 0; l < width; ++l)
            v[l] = v[l] + v[l + width];
    float result = v[0];
    for (; i < count; ++i)
        result += a[i] * b[i];
    return result;
}

void orc_sdpa_head(const float* query, const float* key, const float* value, float* output,
                   int query_tokens, int key_tokens, int key_dim, int value_dim, float scale,
                   const float* mask) {
    float* scores = (float*)malloc(sizeof(float) * (size_t)(key_tokens > 0 ? key_tokens : 1));
    for (int t = 0; t < query_tokens; ++t) {
        const float* q = query + (size_t)t * key_dim;
        const float* mrow = mask ? mask + (size_t)t * key_tokens : NULL;
        int visible = key_tokens;
        if (mrow)
            while (visible > 0 && mrow[visible - 1] == -INFINITY)
                --visible;
        float* o = output + (size_t)t * value_dim;
        memset(o, 0, sizeof(float) * (size_t)value_dim);
        if (visible == 0)
            continue;
        for (int j = 0; j < visible; ++j) {
            scores[j] = orc_dot_avx512(q, key + (size_t)j * key_dim, key_dim) * scale;
            if (mrow)
                scores[j] += mrow[j];
        }
        float maximum = -INFINITY;
        for (int j = 0; j < visible; ++j)
            maximum = scores[j] > maximum ? scores[j] : maximum;
        float sum = 0.0f;
        for (int j = 0; j < visible; ++j) {
            scores[j] = orc_exp(scores[j] - maximum);
            sum += scores[j];
        }
        float inverse = 1.0f / sum;
        for (int j = 0; j < visible; ++j)
            scores[j] *= inverse;
        for (int j = 0; j < visible; ++j) {
            float p = scores[j];
            if (p == 0.0f)
                continue;
            const float* vr = value + (size_t)j * value_dim;
            for (int d = 0; d < value_dim; ++d)
                o[d] = fmaf(vr[d], p, o[d]);
        }
    }
    free(scores);
}


/* ------------------------------------------- routing, the other score kinds --
 * kernels/moe_routing.cpp:25-169 beyond the softmax case: score kind 1 takes the logistic
 * function of each logit, kind 2 the square root of softplus (:10-22); an optional per-expert
 * bias is added for the CHOICE only (:72-73); with expert groups, a group is scored by the
 * sum of its two best choice scores (the best alone if it has one expert), the best
 * `topk_groups` groups stay -- insertion with strict '>', so the lower group id wins ties --
 * and the experts of the other groups drop out (:76-122); the top k choice scores are taken
 * as in the softmax case; the weights are the UNBIASED scores of the chosen experts, divided
 * by their sum when asked (0 if the sum is not positive), times a scaling factor (:146-156).
 * Score kind 0 is orc_moe_select_routes_softmax.                                            */

static float score_logistic(float v) { return 1.0f / (1.0f + orc_exp(-v)); }

static float score_sqrt_softplus(float v) {
    float sp = v > 0.0f ? v + log1pf(orc_exp(-v)) : log1pf(orc_exp(v));
    return sqrtf(sp);
}

int orc_moe_select_routes(const float* logits, int tokens, int num_experts, int top_k,
                          int score_kind, int normalize, int groups, int topk_groups,
                          float scaling, const float* bias, int32_t* indices, float* weights) {
    if (score_kind == 0)
        return orc_moe_select_routes_softmax(logits, tokens, num_experts, top_k, indices,
                                             weights);
    if (!logits || tokens <= 0 || num_experts <= 0 || top_k <= 0 || top_k > num_experts ||
        score_kind < 0 || score_kind > 2)
        return -1;
    if (groups < 1)
        groups = 1;
    if (topk_groups <= 0 || topk_groups > groups)
        topk_groups = groups;
    int per_group = num_experts / groups;
    float* score = (float*)malloc(sizeof(float) * (size_t)num_experts);
    float* choice = (float*)malloc(sizeof(float) * (size_t)num_experts);
    float* kept_score = (float*)malloc(sizeof(float) * (size_t)topk_groups);
    int* kept_group = (int*)malloc(sizeof(int) * (size_t)topk_groups);
    for (int t = 0; t < tokens; ++t) {
        const float* row = logits + (size_t)t * num_experts;
        int32_t* idx = indices + (size_t)t * top_k;
        float* w = weights + (size_t)t * top_k;
        for (int e = 0; e < num_experts; ++e) {
            score[e] = score_kind == 1 ? score_logistic(row[e]) : score_sqrt_softplus(row[e]);
            choice[e] = score[e] + (bias ? bias[e] : 0.0f);
        }
        if (groups > 1 && per_group > 0 && topk_groups < groups) {
            for (int j = 0; j < topk_groups; ++j) {
                kept_score[j] = -INFINITY;
                kept_group[j] = 0;
            }
            for (int g = 0; g < groups; ++g) {
                int lo = g * per_group;
                int hi = g == groups - 1 ? num_experts : lo + per_group;
                float first = -INFINITY, second = -INFINITY;
                for (int e = lo; e < hi; ++e) {
                    if (choice[e] > first) {
                        second = first;
                        first = choice[e];
                    } else if (choice[e] > second) {
                        second = choice[e];
                    }
                }
                float gs = isfinite(second) ? first + second : first;
                for (int j = 0; j < topk_groups; ++j) {
                    if (gs > kept_score[j]) {
                        for (int s = topk_groups - 1; s > j; --s) {
                            kept_score[s] = kept_score[s - 1];
                            kept_group[s] = kept_group[s - 1];
                        }
                        kept_score[j] = gs;
                        kept_group[j] = g;
                        break;
                    }
                }
            }
            for (int e = 0; e < num_experts; ++e) {
                int g = e / per_group;
                if (g > groups - 1)
                    g = groups - 1;
                int kept = 0;
                for (int j = 0; j < topk_groups; ++j)
                    kept |= kept_group[j] == g;
                if (!kept)
                    choice[e] = -INFINITY;
            }
        }
        for (int j = 0; j < top_k; ++j) {
            idx[j] = 0;
            w[j] = -INFINITY;
        }
        for (int e = 0; e < num_experts; ++e) {
            float v = choice[e];
            for (int j = 0; j < top_k; ++j) {
                if (v > w[j]) {
                    for (int s = top_k - 1; s > j; --s) {
                        w[s] = w[s - 1];
                        idx[s] = idx[s - 1];
                    }
                    w[j] = v;
                    idx[j] = e;
                    break;
                }
            }
        }
        float sum = 0.0f;
        for (int j = 0; j < top_k; ++j) {
            w[j] = score[idx[j]];
            sum += w[j];
        }
        if (normalize) {
            float inverse = sum > 0.0f ? 1.0f / sum : 0.0f;
            for (int j = 0; j < top_k; ++j)
                w[j] *= inverse;
        }
        for (int j = 0; j < top_k; ++j)
            w[j] *= scaling;
    }
    free(score);
    free(choice);
    free(kept_score);
    free(kept_group);
    return 0;
}

/* ---------------------------------------------------------- rotary tables --
 * engine/input_prep.cpp:18-31 (fill_rope_cache): per position and feature pair i,
 * theta_i = 1 / pow(rope_theta, 2 i / rope_dim), angle = position * theta_i, cos and sin of
 * the angle -- all float, through the host libm (std::pow / std::cos / std::sin on floats are
 * powf / cosf / sinf).  cos_out / sin_out: [positions][rope_dim / 2].                        */
void orc_rope_tables(float* cos_out, float* sin_out, int positions, int first_position,
                     int rope_dim, float rope_theta) {
    const int half = rope_dim / 2;
    for (int n = 0; n < positions; ++n) {
        const int pos = first_position + n;
        for (int i = 0; i < half; ++i) {
            const float theta = 1.0f / powf(rope_theta, 2.0f * i / rope_dim);
            const float angle = pos * theta;
            cos_out[(size_t)n * half + i] = cosf(angle);
            sin_out[(size_t)n * half + i] = sinf(angle);
        }
    }
}
