// Mixture of experts, the steps between the two products.
//
// The experts' gate and up projections run as ONE product over all experts (rows [gate_0; up_0; gate_1; up_1; ...; then the
// shared expert's gate and up]), and the down projections as ONE product whose input is every expert's activation side by
// side: an expert that a token did not choose contributes an activation of exactly zero, a chosen one its activation times
// its routing weight.  This kernel makes that input: per token it turns the router's logits into weights (softmax over all
// experts in 32-bit, the `top` largest scores keep their value, the others become 0; ties go to the lower index) and writes
//     y[t, e, i] = weight[t, e] * g * sigmoid(alpha * g) * (u + 1),   g = min(gate, limit), u = clamp(up, -limit, limit)
// for every expert, and the same with the weight sigmoid(shared gate logit) and its own limit for the shared expert.
//
// Options of the routing (MoeRouting; all off by default): the router may have more outputs than there are experts, the last
// `identity` of them standing for experts whose output is the token's input itself (the sum of the chosen ones' weights goes
// to id_weight[t], and the caller adds id_weight[t] * input[t]); a `correction` vector is added to the scores for the CHOICE
// only (the weights stay the plain scores); the outputs form `group_count` equal groups of neighbours, a group's score is its
// largest choice score, and only the outputs of the `group_keep` best groups can be chosen.  `act` 1: an expert is
// weight * silu(gate) * up, without clamps.
#include "common.cuh"

SPY_MODULE(spy_moe)

constexpr int MOE_MAX_EXPERTS = 1024;

struct MoeRouting {
    int identity;                  // router outputs behind the experts' that stand for identity experts
    const float* correction;       // null, or [experts + identity]: added to the scores for the choice
    int group_count, group_keep;   // 0: no groups
    int act;                       // 0: clamped g * sigmoid(alpha g) * (u + 1); 1: silu(g) * u
    float* id_weight;              // null, or [T]: the sum of the chosen identity experts' weights
    float* shared_weight;          // null, or [T]: the shared expert's weight (sigmoid of its gate's logit)
};

template <typename TA, typename TO>
__global__ void moe_activation_kernel(const TA* __restrict__ gu, long long gu_ld, const float* __restrict__ logits, long long logits_ld,
                                      TO* __restrict__ y, long long y_ld, int experts, int top, int ff, float limit, int shared_ff, float shared_limit,
                                      float alpha, float* __restrict__ weights_out, int vec, MoeRouting r)
{
    extern __shared__ float w_s[];                 // total scores, the shared weight, total kept weights, total choice scores, the groups' scores
    __shared__ float scratch[33];
    pdl_enter();
    const int t = blockIdx.x, tid = threadIdx.x;
    const int total = experts + r.identity;        // the router's outputs; the shared gate's logit lies behind them
    const float* lg = logits + (long long)t * logits_ld;
    float* kept_w = w_s + total + 1;               // kept_w[e]: the weight if chosen, else 0
    float* choice = kept_w + total;                // the score the choice goes by
    float* group_s = choice + total;
    // softmax over all outputs
    float m = -INFINITY;
    for (int e = tid; e < total; e += blockDim.x) m = fmaxf(m, lg[e]);
    m = block_max(m, scratch);
    float s = 0.f;
    for (int e = tid; e < total; e += blockDim.x) s += expf(lg[e] - m);
    s = block_sum(s, scratch);
    for (int e = tid; e < total; e += blockDim.x) {
        const float v = expf(lg[e] - m) / s;
        w_s[e] = v;
        choice[e] = r.correction != nullptr ? v + r.correction[e] : v;
    }
    __syncthreads();
    if (r.group_count > 0) {
        // a group's score is its largest choice score; a group stays when fewer than group_keep groups beat it
        const int per = total / r.group_count;
        for (int g = tid; g < r.group_count; g += blockDim.x) {
            float best = -INFINITY;
            for (int e = g * per; e < g * per + per; ++e) best = fmaxf(best, choice[e]);
            group_s[g] = best;
        }
        __syncthreads();
        for (int e = tid; e < total; e += blockDim.x) {
            const int g = e / per;
            const float v = group_s[g];
            int ahead = 0;
            for (int o = 0; o < r.group_count; ++o) {
                const float x = group_s[o];
                ahead += (x > v || (x == v && o < g)) ? 1 : 0;
            }
            if (ahead >= r.group_keep) choice[e] = -INFINITY;
        }
        __syncthreads();
    }
    // the `top` largest stay: an output stays when fewer than `top` beat it (a larger choice score, or an equal one at a lower index)
    for (int e = tid; e < total; e += blockDim.x) {
        const float v = choice[e];
        int ahead = 0;
        for (int o = 0; o < total; ++o) {
            const float x = choice[o];
            ahead += (x > v || (x == v && o < e)) ? 1 : 0;
        }
        kept_w[e] = (ahead < top && v > -INFINITY) ? w_s[e] : 0.f;
    }
    if (tid == 0) w_s[total] = shared_ff > 0 ? 1.0f / (1.0f + expf(-lg[total])) : 0.f;
    __syncthreads();
    if (r.id_weight != nullptr && tid == 0) {
        float idw = 0.f;
        for (int e = experts; e < total; ++e) idw += kept_w[e];
        r.id_weight[t] = idw;
    }
    if (r.shared_weight != nullptr && tid == 0) r.shared_weight[t] = w_s[total];
    if (weights_out != nullptr)
        for (int e = tid; e <= total; e += blockDim.x) weights_out[(long long)t * (total + 1) + e] = e < total ? kept_w[e] : w_s[total];
    if (gu == nullptr) return;                   // the weights alone were asked for
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
                if (i < routed) { const int e = i / ff; j = i - e * ff; n = ff; w = kept_w[e]; lim = limit; src = g_row + (long long)e * 2 * ff; }
                else { j = i - routed; n = shared_ff; w = w_s[total]; lim = shared_limit; src = g_row + (long long)routed * 2; }
                uint4 packed = make_uint4(0u, 0u, 0u, 0u);
                if (w != 0.f) {
                    const uint4 gq = *reinterpret_cast<const uint4*>(src + j), uq = *reinterpret_cast<const uint4*>(src + n + j);
                    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gq);
                    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uq);
                    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (r.act == 1) {
                            const float ga = __low2float(g2[q]), gb = __high2float(g2[q]);
                            o2[q] = __floats2bfloat162_rn(w * (ga / (1.0f + expf(-ga))) * __low2float(u2[q]), w * (gb / (1.0f + expf(-gb))) * __high2float(u2[q]));
                            continue;
                        }
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
        if (i < routed) { const int e = i / ff; j = i - e * ff; n = ff; w = kept_w[e]; lim = limit; src = g_row + (long long)e * 2 * ff; }
        else { j = i - routed; n = shared_ff; w = w_s[total]; lim = shared_limit; src = g_row + (long long)routed * 2; }
        float res = 0.f;
        if (w != 0.f && r.act == 1) {
            const float g = to_f32(src[j]);
            res = w * (g / (1.0f + expf(-g))) * to_f32(src[n + j]);
        } else if (w != 0.f) {
            const float g = fminf(to_f32(src[j]), lim);
            const float u = fminf(fmaxf(to_f32(src[n + j]), -lim), lim);
            res = w * (g / (1.0f + expf(-alpha * g))) * (u + 1.0f);
        }
        y_row[i] = from_f32<TO>(res);
    }
}

// gu [T, gu_ld]: per expert [gate (ff) | up (ff)], then the shared expert's [gate (shared_ff) | up (shared_ff)];
// logits [T, logits_ld] float32: the router's `experts` logits, then (with a shared expert) the shared gate's logit;
// y [T, y_ld]: experts * ff + shared_ff columns; weights_out (optional) [T, experts + identity + 1] float32 receives the weights.
static int run_moe_activation(const void* gu, int gu_dtype, long long gu_ld, const float* logits, long long logits_ld, void* y, int y_dtype,
                              long long y_ld, int tokens, int experts, int top, int ff, float limit, int shared_ff, float shared_limit, float alpha,
                              float* weights_out, MoeRouting r, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    const int total = experts + r.identity;
    if (experts <= 0 || r.identity < 0 || total > MOE_MAX_EXPERTS || top <= 0 || top > total || ff <= 0 || shared_ff < 0)
        SPY_FAIL("moe_activation: %d experts and %d identity experts (at most %d), top %d, expert size %d, shared size %d", experts, r.identity,
                 MOE_MAX_EXPERTS, top, ff, shared_ff);
    if (r.group_count < 0 || (r.group_count > 0 && (total % r.group_count != 0 || r.group_keep <= 0 || r.group_keep > r.group_count
                                                    || (long long)r.group_keep * (total / r.group_count) < top)))
        SPY_FAIL("moe_activation: %d groups of which %d are kept do not fit %d router outputs and top %d", r.group_count, r.group_keep, total, top);
    if (r.act < 0 || r.act > 1) SPY_FAIL("moe_activation: activation code %d", r.act);
    const size_t smem = (size_t)(3 * total + 1 + (r.group_count > 0 ? r.group_count : 0)) * sizeof(float);
    const int vec = gu_dtype == SPY_BF16 && y_dtype == SPY_BF16 && ff % 8 == 0 && shared_ff % 8 == 0 && gu_ld % 8 == 0 && y_ld % 8 == 0
                    && ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    SPY_DISPATCH_DTYPE(gu_dtype, TA, {
        SPY_DISPATCH_DTYPE(y_dtype, TO, {
            spy_launch(moe_activation_kernel<TA, TO>, dim3(tokens), dim3(256), smem, stream, (const TA*)gu, gu_ld, logits, logits_ld, (TO*)y, y_ld,
                       experts, top, ff, limit, shared_ff, shared_limit, alpha, weights_out, vec, r);
        })
    })
    SPY_CHECK_LAUNCH("moe_activation");
    return 0;
}

extern "C" int spy_moe_activation(const void* gu, int gu_dtype, long long gu_ld, const float* logits, long long logits_ld, void* y, int y_dtype,
                                  long long y_ld, int tokens, int experts, int top, int ff, float limit, int shared_ff, float shared_limit, float alpha,
                                  float* weights_out, cudaStream_t stream)
{
    MoeRouting r = {0, nullptr, 0, 0, 0, nullptr, nullptr};
    return run_moe_activation(gu, gu_dtype, gu_ld, logits, logits_ld, y, y_dtype, y_ld, tokens, experts, top, ff, limit, shared_ff, shared_limit, alpha,
                              weights_out, r, stream);
}

// The same with the routing's options (see the head of this file); logits hold experts + identity columns, then the shared gate's.
// gu null (y then unused): the routing alone, its weights into weights_out, id_weight and shared_weight.
extern "C" int spy_moe_activation_routed(const void* gu, int gu_dtype, long long gu_ld, const float* logits, long long logits_ld, void* y, int y_dtype,
                                         long long y_ld, int tokens, int experts, int top, int ff, float limit, int shared_ff, float shared_limit,
                                         float alpha, float* weights_out, int identity, const float* correction, int group_count, int group_keep, int act,
                                         float* id_weight, float* shared_weight, cudaStream_t stream)
{
    if (gu == nullptr && weights_out == nullptr) SPY_FAIL("moe_activation: neither activations nor weights are asked for");
    MoeRouting r = {identity, correction, group_count, group_keep, act, id_weight, shared_weight};
    return run_moe_activation(gu, gu_dtype, gu_ld, logits, logits_ld, y, y_dtype, y_ld, tokens, experts, top, ff, limit, shared_ff, shared_limit, alpha,
                              weights_out, r, stream);
}

// out[t, :] += w[t] * x[t, :] in 32-bit (out float32): what the identity experts of a mixture contribute.
template <typename TX>
__global__ void add_scaled_rows_kernel(float* __restrict__ out, const TX* __restrict__ x, const float* __restrict__ w, int width, long long total)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const float wt = w[i / width];
        if (wt != 0.f) out[i] = fmaf(wt, to_f32(x[i]), out[i]);
    }
}

extern "C" int spy_add_scaled_rows(float* out, const void* x, int x_dtype, const float* w, int tokens, int width, cudaStream_t stream)
{
    if (tokens <= 0 || width <= 0) return 0;
    const long long total = (long long)tokens * width;
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    SPY_DISPATCH_DTYPE(x_dtype, TX, {
        spy_launch(add_scaled_rows_kernel<TX>, dim3((int)blocks), dim3(256), 0, stream, out, (const TX*)x, w, width, total);
    })
    SPY_CHECK_LAUNCH("add_scaled_rows");
    return 0;
}

// ---- the routed form, for steps of many tokens ------------------------------------------------------------------------
//
// With many tokens a step, computing every expert for every token wastes experts / top of the products.  The routed form
// sorts the (token, chosen expert) pairs by expert, gathers the tokens' rows in that order, runs each expert's products on
// its own run of rows, and adds each token's `top` results up again in a fixed order.  The weights are the same as above
// (moe_route repeats the softmax and the choice), so a token's result differs from the dense form by rounding only.

// One warp a token (a block walks over tokens with a stride): the chosen experts in ascending order with their weights, the shared
// expert's gate, and the experts' counts (added up per block in shared memory first, so few additions meet in global memory).
__global__ void moe_route_kernel(const float* __restrict__ logits, long long logits_ld, int tokens, int experts, int top, int has_shared,
                                 int* __restrict__ choice, float* __restrict__ choice_w, float* __restrict__ shared_w, int* __restrict__ counts)
{
    extern __shared__ float w_all[];               // experts floats a warp, then the block's counts
    pdl_enter();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    int* hist = reinterpret_cast<int*>(w_all + (long long)nwarps * experts);
    for (int e = threadIdx.x; e < experts; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    float* w_s = w_all + (long long)warp * experts;
    for (long long t = (long long)blockIdx.x * nwarps + warp; t < tokens; t += (long long)gridDim.x * nwarps) {
        const float* lg = logits + t * logits_ld;
        float m = -INFINITY;
        for (int e = lane; e < experts; e += 32) m = fmaxf(m, lg[e]);
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float s = 0.f;
        for (int e = lane; e < experts; e += 32) s += expf(lg[e] - m);
        s = warp_sum(s);
        __syncwarp();
        for (int e = lane; e < experts; e += 32) w_s[e] = expf(lg[e] - m) / s;
        __syncwarp();
        int k_base = 0;
        for (int e0 = 0; e0 < experts; e0 += 32) {
            const int e = e0 + lane;
            bool chosen = false;
            float v = 0.f;
            if (e < experts) {
                v = w_s[e];
                int ahead = 0;
                for (int o = 0; o < experts; ++o) {
                    const float x = w_s[o];
                    ahead += (x > v || (x == v && o < e)) ? 1 : 0;
                }
                chosen = ahead < top;
            }
            const unsigned ballot = __ballot_sync(0xffffffffu, chosen);
            if (chosen) {
                const int k = k_base + __popc(ballot & ((1u << lane) - 1u));
                choice[t * top + k] = e;
                choice_w[t * top + k] = v;
                atomicAdd(hist + e, 1);
            }
            k_base += __popc(ballot);
        }
        if (lane == 0 && has_shared) shared_w[t] = 1.0f / (1.0f + expf(-lg[experts]));
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
        if (hist[e] != 0) atomicAdd(counts + e, hist[e]);
}

// One block an expert: its rows' places, in the order of the tokens.  Each warp takes a run of the pairs, counts the expert's
// pairs in it, and after a prefix over the warps' counts hands out the places.  offsets [experts + 1]; slot [tokens * top]: the
// row of each (token, k); row_token, row_w [tokens * top]: each row's token and weight.
__global__ void __launch_bounds__(1024)
moe_slots_kernel(const int* __restrict__ choice, const float* __restrict__ choice_w, const int* __restrict__ counts, int pairs,
                 int top, int experts, int* __restrict__ offsets, int* __restrict__ slot, int* __restrict__ row_token,
                 float* __restrict__ row_w)
{
    __shared__ int warp_count[32];
    __shared__ int first_row;
    pdl_enter();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int e = blockIdx.x;
    const int per_warp = ((pairs + nwarps - 1) / nwarps + 31) / 32 * 32;
    const int i_first = min(warp * per_warp, pairs), i_end = min(i_first + per_warp, pairs);
    int mine_count = 0;
    for (int i0 = i_first; i0 < i_end; i0 += 32) {
        const int i = i0 + lane;
        mine_count += __popc(__ballot_sync(0xffffffffu, i < i_end && choice[i] == e));
    }
    if (lane == 0) warp_count[warp] = mine_count;
    if (warp == 0) {
        int base = 0;
        for (int o = lane; o < e; o += 32) base += counts[o];
        for (int o = 16; o > 0; o >>= 1) base += __shfl_xor_sync(0xffffffffu, base, o);
        if (lane == 0) {
            first_row = base;
            offsets[e] = base;
            if (e == experts - 1) offsets[experts] = base + counts[e];
        }
    }
    __syncthreads();
    int base = first_row;
    for (int w = 0; w < warp; ++w) base += warp_count[w];
    for (int i0 = i_first; i0 < i_end; i0 += 32) {
        const int i = i0 + lane;
        const bool mine = i < i_end && choice[i] == e;
        const unsigned ballot = __ballot_sync(0xffffffffu, mine);
        if (mine) {
            const int r = base + __popc(ballot & ((1u << lane) - 1u));
            slot[i] = r;
            row_token[r] = i / top;
            row_w[r] = choice_w[i];
        }
        base += __popc(ballot);
    }
}

// out[r] = in[row_token[r]]: rows of `len` elements of 2 bytes (bf16) or 4, copied 16 bytes at a time where the rows allow it.
__global__ void gather_rows_kernel(const uint8_t* __restrict__ in, const int* __restrict__ row_token, uint8_t* __restrict__ out, long long row_bytes)
{
    pdl_enter();
    const uint8_t* src = in + (long long)row_token[blockIdx.x] * row_bytes;
    uint8_t* dst = out + (long long)blockIdx.x * row_bytes;
    if ((row_bytes & 15) == 0) {
        for (long long i = threadIdx.x * 16LL; i < row_bytes; i += blockDim.x * 16LL) *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
    } else {
        for (long long i = threadIdx.x; i < row_bytes; i += blockDim.x) dst[i] = src[i];
    }
}

// y[r, i] = w[r] * g * sigmoid(alpha g) * (u + 1) over rows of [gate (ff) | up (ff)], g = min(gate, limit), u = clamp(up, -limit, limit)
template <typename TA, typename TO>
__global__ void expert_activation_kernel(const TA* __restrict__ gu, long long gu_ld, const float* __restrict__ row_w, TO* __restrict__ y, long long y_ld,
                                         int ff, float limit, float alpha, int vec, int act)
{
    pdl_enter();
    const long long r = blockIdx.x;
    const float w = row_w[r];
    const TA* src = gu + r * gu_ld;
    TO* dst = y + r * y_ld;
    if constexpr (sizeof(TA) == 2 && sizeof(TO) == 2) {
        if (vec) {                                  // eight elements (16 bytes) a thread and step
            for (int i = threadIdx.x * 8; i < ff; i += blockDim.x * 8) {
                const uint4 gq = *reinterpret_cast<const uint4*>(src + i), uq = *reinterpret_cast<const uint4*>(src + ff + i);
                const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gq);
                const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uq);
                uint4 packed;
                __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    if (act == 1) {
                        const float ga = __low2float(g2[q]), gb = __high2float(g2[q]);
                        o2[q] = __floats2bfloat162_rn(w * (ga / (1.0f + expf(-ga))) * __low2float(u2[q]), w * (gb / (1.0f + expf(-gb))) * __high2float(u2[q]));
                        continue;
                    }
                    const float ga = fminf(__low2float(g2[q]), limit), gb = fminf(__high2float(g2[q]), limit);
                    const float ua = fminf(fmaxf(__low2float(u2[q]), -limit), limit), ub = fminf(fmaxf(__high2float(u2[q]), -limit), limit);
                    o2[q] = __floats2bfloat162_rn(w * (ga / (1.0f + expf(-alpha * ga))) * (ua + 1.0f), w * (gb / (1.0f + expf(-alpha * gb))) * (ub + 1.0f));
                }
                *reinterpret_cast<uint4*>(dst + i) = packed;
            }
            return;
        }
    }
    for (int i = threadIdx.x; i < ff; i += blockDim.x) {
        if (act == 1) {
            const float g = to_f32(src[i]);
            dst[i] = from_f32<TO>(w * (g / (1.0f + expf(-g))) * to_f32(src[ff + i]));
            continue;
        }
        const float g = fminf(to_f32(src[i]), limit);
        const float u = fminf(fmaxf(to_f32(src[ff + i]), -limit), limit);
        dst[i] = from_f32<TO>(w * (g / (1.0f + expf(-alpha * g))) * (u + 1.0f));
    }
}

// out[t] = sum over k (ascending) of rows[slot[t, k]] (+ shared[t]); rows and shared float32 or bf16, out float32
template <typename TR>
__global__ void moe_combine_kernel(const TR* __restrict__ rows, const int* __restrict__ slot, int top, const TR* __restrict__ shared, float* __restrict__ out, int len)
{
    pdl_enter();
    const long long t = blockIdx.x;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int r = slot[t * top + k];         // below 0: the pair has no row (fewer experts than `top` were chosen)
            if (r >= 0) acc += to_f32(rows[(long long)r * len + i]);
        }
        if (shared != nullptr) acc += to_f32(shared[t * len + i]);
        out[t * len + i] = acc;
    }
}

extern "C" int spy_moe_route(const float* logits, long long logits_ld, int tokens, int experts, int top, int has_shared, int* choice, float* choice_w,
                             float* shared_w, int* counts, int* offsets, int* slot, int* row_token, float* row_w, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0 || top > experts) SPY_FAIL("moe_route: %d experts (at most %d), top %d", experts, MOE_MAX_EXPERTS, top);
    SPY_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * experts, stream));
    const int warps = 4;
    const int blocks = min((tokens + warps - 1) / warps, 4 * 148);
    spy_launch_in_order(moe_route_kernel, dim3(blocks), dim3(32 * warps), ((size_t)warps * experts + experts) * sizeof(float), stream, logits, logits_ld,
                        tokens, experts, top, has_shared, choice, choice_w, shared_w, counts);
    SPY_CHECK_LAUNCH("moe_route");
    spy_launch(moe_slots_kernel, dim3(experts), dim3(1024), 0, stream, (const int*)choice, (const float*)choice_w, (const int*)counts,
               tokens * top, top, experts, offsets, slot, row_token, row_w);
    SPY_CHECK_LAUNCH("moe_slots");
    return 0;
}

// The (token, chosen expert) pairs of a step from a matrix of routing weights [tokens, ld] whose entry is the expert's weight where
// the token chose it and 0 elsewhere (what moe_activation leaves in weights_out): a token's chosen experts in ascending order, at
// most `top` of them; pairs beyond a token's last have the expert -1, weight 0 and no row.  One warp a token.
__global__ void moe_pairs_kernel(const float* __restrict__ weights, long long ld, int tokens, int experts, int top, int* __restrict__ choice,
                                 float* __restrict__ choice_w, int* __restrict__ slot, int* __restrict__ counts)
{
    extern __shared__ int hist_s[];
    pdl_enter();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) hist_s[e] = 0;
    __syncthreads();
    for (long long t = (long long)blockIdx.x * nwarps + warp; t < tokens; t += (long long)gridDim.x * nwarps) {
        const float* w = weights + t * ld;
        int k_base = 0;
        for (int e0 = 0; e0 < experts; e0 += 32) {
            const int e = e0 + lane;
            const float v = e < experts ? w[e] : 0.f;
            const bool chosen = v != 0.f;
            const unsigned ballot = __ballot_sync(0xffffffffu, chosen);
            const int k = k_base + __popc(ballot & ((1u << lane) - 1u));
            if (chosen && k < top) {
                choice[t * top + k] = e;
                choice_w[t * top + k] = v;
                atomicAdd(hist_s + e, 1);
            }
            k_base += __popc(ballot);
        }
        for (int k = min(k_base, top) + lane; k < top; k += 32) {
            choice[t * top + k] = -1;
            choice_w[t * top + k] = 0.f;
        }
        for (int k = lane; k < top; k += 32) slot[t * top + k] = -1;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
        if (hist_s[e] != 0) atomicAdd(counts + e, hist_s[e]);
}

// weights [tokens, ld] float32 (the first `experts` columns are looked at); the other arrays as for spy_moe_route.
extern "C" int spy_moe_route_weights(const float* weights, long long ld, int tokens, int experts, int top, int* choice, float* choice_w, int* counts,
                                     int* offsets, int* slot, int* row_token, float* row_w, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0) SPY_FAIL("moe_route_weights: %d experts (at most %d), top %d", experts, MOE_MAX_EXPERTS, top);
    SPY_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * experts, stream));
    const int warps = 4;
    const int blocks = min((tokens + warps - 1) / warps, 4 * 148);
    spy_launch_in_order(moe_pairs_kernel, dim3(blocks), dim3(32 * warps), (size_t)experts * sizeof(int), stream, weights, ld, tokens, experts, top, choice,
                        choice_w, slot, counts);
    SPY_CHECK_LAUNCH("moe_pairs");
    spy_launch(moe_slots_kernel, dim3(experts), dim3(1024), 0, stream, (const int*)choice, (const float*)choice_w, (const int*)counts,
               tokens * top, top, experts, offsets, slot, row_token, row_w);
    SPY_CHECK_LAUNCH("moe_slots");
    return 0;
}

extern "C" int spy_gather_rows(const void* in, const int* row_token, void* out, int rows, long long row_bytes, cudaStream_t stream)
{
    if (rows <= 0 || row_bytes <= 0) return 0;
    spy_launch(gather_rows_kernel, dim3(rows), dim3(128), 0, stream, (const uint8_t*)in, row_token, (uint8_t*)out, row_bytes);
    SPY_CHECK_LAUNCH("gather_rows");
    return 0;
}

// act: 0 the clamped form above, 1 w * silu(gate) * up without clamps
extern "C" int spy_expert_activation(const void* gu, int gu_dtype, long long gu_ld, const float* row_w, void* y, int y_dtype, long long y_ld, int rows, int ff,
                                     float limit, float alpha, cudaStream_t stream, int act)
{
    if (rows <= 0 || ff <= 0) return 0;
    if (act < 0 || act > 1) SPY_FAIL("expert_activation: activation code %d", act);
    const int vec = gu_dtype == SPY_BF16 && y_dtype == SPY_BF16 && ff % 8 == 0 && gu_ld % 8 == 0 && y_ld % 8 == 0
                    && ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    SPY_DISPATCH_DTYPE(gu_dtype, TA, {
        SPY_DISPATCH_DTYPE(y_dtype, TO, {
            spy_launch(expert_activation_kernel<TA, TO>, dim3(rows), dim3(256), 0, stream, (const TA*)gu, gu_ld, row_w, (TO*)y, y_ld, ff, limit, alpha, vec, act);
        })
    })
    SPY_CHECK_LAUNCH("expert_activation");
    return 0;
}

extern "C" int spy_moe_combine(const void* rows, int rows_dtype, const int* slot, int top, const void* shared, float* out, int tokens, int len, cudaStream_t stream)
{
    if (tokens <= 0 || len <= 0) return 0;
    SPY_DISPATCH_DTYPE(rows_dtype, TR, {
        spy_launch(moe_combine_kernel<TR>, dim3(tokens), dim3(256), 0, stream, (const TR*)rows, slot, top, (const TR*)shared, out, len);
    })
    SPY_CHECK_LAUNCH("moe_combine");
    return 0;
}
