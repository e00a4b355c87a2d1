// Mixture of experts, the steps between the two products.
//
// The experts' gate and up projections run as ONE product over all experts (rows [gate_0; up_0; gate_1; up_1; ...; then the
// shared expert's gate and up]), and the down projections as ONE product whose input is every expert's activation side by
// side: an expert that a token did not choose contributes an activation of exactly zero, a chosen one its activation times
// its routing weight.  This kernel makes that input: per token it turns the router's logits into weights (softmax over all
// experts in 32-bit, the `top` largest scores keep their value, the others become 0; ties go to the lower index) and writes
//     y[t, e, i] = weight[t, e] * g * sigmoid(alpha * g) * (u + 1),   g = min(gate, limit), u = clamp(up, -limit, limit)
// for every expert, and the same with the weight sigmoid(shared gate logit) and its own limit for the shared expert.
#include "common.cuh"

SPY_MODULE(spy_moe)

constexpr int MOE_MAX_EXPERTS = 1024;

template <typename TA, typename TO>
__global__ void moe_activation_kernel(const TA* __restrict__ gu, long long gu_ld, const float* __restrict__ logits, long long logits_ld,
                                      TO* __restrict__ y, long long y_ld, int experts, int top, int ff, float limit, int shared_ff, float shared_limit,
                                      float alpha, float* __restrict__ weights_out, int vec)
{
    extern __shared__ float w_s[];                 // experts + 1 weights
    __shared__ float scratch[33];
    pdl_enter();
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* lg = logits + (long long)t * logits_ld;
    // softmax over all experts
    float m = -INFINITY;
    for (int e = tid; e < experts; e += blockDim.x) m = fmaxf(m, lg[e]);
    m = block_max(m, scratch);
    float s = 0.f;
    for (int e = tid; e < experts; e += blockDim.x) s += expf(lg[e] - m);
    s = block_sum(s, scratch);
    for (int e = tid; e < experts; e += blockDim.x) w_s[e] = expf(lg[e] - m) / s;
    __syncthreads();
    // the `top` largest stay: an expert stays when fewer than `top` experts beat it (a larger score, or an equal one at a lower index)
    for (int e = tid; e < experts; e += blockDim.x) {
        const float v = w_s[e];
        int ahead = 0;
        for (int o = 0; o < experts; ++o) {
            const float x = w_s[o];
            ahead += (x > v || (x == v && o < e)) ? 1 : 0;
        }
        w_s[experts + 1 + e] = ahead < top ? v : 0.f;
    }
    if (tid == 0) w_s[experts] = shared_ff > 0 ? 1.0f / (1.0f + expf(-lg[experts])) : 0.f;
    __syncthreads();
    if (weights_out != nullptr)
        for (int e = tid; e <= experts; e += blockDim.x) weights_out[(long long)t * (experts + 1) + e] = e < experts ? w_s[experts + 1 + e] : w_s[experts];
    const TA* g_row = gu + (long long)t * gu_ld;
    TO* y_row = y + (long long)t * y_ld;
    const int routed = experts * ff;
    if constexpr (sizeof(TA) == 2 && sizeof(TO) == 2) {
        if (vec) {
            // eight elements (16 bytes) a thread and step; a run of eight lies within one expert, and an expert that the token did
            // not choose costs one store of zeros and no load
            for (int i = tid * 8; i < routed + shared_ff; i += blockDim.x * 8) {
                float w, lim;
                const TA* src;
                int j, n;
                if (i < routed) { const int e = i / ff; j = i - e * ff; n = ff; w = w_s[experts + 1 + e]; lim = limit; src = g_row + (long long)e * 2 * ff; }
                else { j = i - routed; n = shared_ff; w = w_s[experts]; lim = shared_limit; src = g_row + (long long)routed * 2; }
                uint4 packed = make_uint4(0u, 0u, 0u, 0u);
                if (w != 0.f) {
                    const uint4 gq = *reinterpret_cast<const uint4*>(src + j), uq = *reinterpret_cast<const uint4*>(src + n + j);
                    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gq);
                    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uq);
                    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float ga = fminf(__low2float(g2[q]), lim), gb = fminf(__high2float(g2[q]), lim);
                        const float ua = fminf(fmaxf(__low2float(u2[q]), -lim), lim), ub = fminf(fmaxf(__high2float(u2[q]), -lim), lim);
                        o2[q] = __floats2bfloat162_rn(w * (ga / (1.0f + expf(-alpha * ga))) * (ua + 1.0f), w * (gb / (1.0f + expf(-alpha * gb))) * (ub + 1.0f));
                    }
                }
                *reinterpret_cast<uint4*>(y_row + i) = packed;
            }
            return;
        }
    }
    for (int i = tid; i < routed + shared_ff; i += blockDim.x) {
        float w, lim;
        const TA* src;
        int j, n;
        if (i < routed) { const int e = i / ff; j = i - e * ff; n = ff; w = w_s[experts + 1 + e]; lim = limit; src = g_row + (long long)e * 2 * ff; }
        else { j = i - routed; n = shared_ff; w = w_s[experts]; lim = shared_limit; src = g_row + (long long)routed * 2; }
        float r = 0.f;
        if (w != 0.f) {
            const float g = fminf(to_f32(src[j]), lim);
            const float u = fminf(fmaxf(to_f32(src[n + j]), -lim), lim);
            r = w * (g / (1.0f + expf(-alpha * g))) * (u + 1.0f);
        }
        y_row[i] = from_f32<TO>(r);
    }
}

// gu [T, gu_ld]: per expert [gate (ff) | up (ff)], then the shared expert's [gate (shared_ff) | up (shared_ff)];
// logits [T, logits_ld] float32: the router's `experts` logits, then (with a shared expert) the shared gate's logit;
// y [T, y_ld]: experts * ff + shared_ff columns; weights_out (optional) [T, experts + 1] float32 receives the weights.
extern "C" int spy_moe_activation(const void* gu, int gu_dtype, long long gu_ld, const float* logits, long long logits_ld, void* y, int y_dtype,
                                  long long y_ld, int tokens, int experts, int top, int ff, float limit, int shared_ff, float shared_limit, float alpha,
                                  float* weights_out, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0 || top > experts || ff <= 0 || shared_ff < 0)
        SPY_FAIL("moe_activation: %d experts (at most %d), top %d, expert size %d, shared size %d", experts, MOE_MAX_EXPERTS, top, ff, shared_ff);
    const size_t smem = (size_t)(2 * experts + 2) * sizeof(float);
    const int vec = gu_dtype == SPY_BF16 && y_dtype == SPY_BF16 && ff % 8 == 0 && shared_ff % 8 == 0 && gu_ld % 8 == 0 && y_ld % 8 == 0
                    && ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    SPY_DISPATCH_DTYPE(gu_dtype, TA, {
        SPY_DISPATCH_DTYPE(y_dtype, TO, {
            spy_launch(moe_activation_kernel<TA, TO>, dim3(tokens), dim3(256), smem, stream, (const TA*)gu, gu_ld, logits, logits_ld, (TO*)y, y_ld,
                       experts, top, ff, limit, shared_ff, shared_limit, alpha, weights_out, vec);
        })
    })
    SPY_CHECK_LAUNCH("moe_activation");
    return 0;
}
