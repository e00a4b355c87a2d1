// Recurrences whose state is a vector (or a small matrix per channel) carried from token to token in each request's slot,
// in 32-bit.  A step brings a run of consecutive tokens for each request; a thread owns one channel (or a share of one
// channel's states) of one request and walks the run in order, so a token's result does not depend on where the run was cut.
//
// mingru_scan:  z = sigmoid(pz + bz), u = px + bx, c = u + 1/2 where u >= 0, sigmoid(u) where u < 0,
//               S <- (1 - z) S + z c,  out = S * silu(pg)                      (element by element over `width` channels)
// selective_scan:  dt = softplus(pdt + bdt), A = -exp(A_log); per channel c and state n
//               S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,  y_c = sum_n S[c, n] C_n + D_c x_c,  out = y * silu(z)
#include "common.cuh"

SPY_MODULE(spy_gated_scan)

__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + expf(-v)); }

constexpr int SCAN_SLICED_FROM = 16;      // a step whose longest run has more tokens than this is scanned in slices

template <typename TB, typename TO>
__global__ void mingru_scan_kernel(const float* __restrict__ proj, long long ld, int z_col, int x_col, int g_col, const TB* __restrict__ z_bias,
                                   const TB* __restrict__ x_bias, float* __restrict__ state, const int* __restrict__ q_start,
                                   const int* __restrict__ state_slot, TO* __restrict__ out, int width)
{
    pdl_enter();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, seq = blockIdx.y;
    const int start = q_start[seq], end = q_start[seq + 1];
    if (c >= width || start >= end) return;
    float* st = state + (long long)state_slot[seq] * width + c;
    float S = *st;
    const float bz = z_bias != nullptr ? to_f32(z_bias[c]) : 0.f, bx = x_bias != nullptr ? to_f32(x_bias[c]) : 0.f;
    const float* p = proj + (long long)start * ld + c;
#pragma unroll 4
    for (int t = start; t < end; ++t, p += ld) {
        const float z = sigmoidf_(p[z_col] + bz);
        const float u = p[x_col] + bx;
        const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
        const float g = p[g_col];
        S = (1.0f - z) * S + z * cand;
        out[(long long)t * width + c] = from_f32<TO>(S * (g * sigmoidf_(g)));
    }
    *st = S;
}

// The same recurrence over long runs, parallel over time: S_t = a_t S_(t-1) + b_t with a = 1 - z, b = z c is linear in S, so a
// run is dealt out in TS consecutive slices, one warp row a slice.  Each slice first folds its tokens into (A, B) with
// S_out = A S_in + B, the slices' (A, B) are chained from the request's state to give every slice its S_in, and each slice
// then walks its tokens again from there in order.  Blocks of 32 channels x TS slices.
template <typename TB, typename TO, int TS>
__global__ void __launch_bounds__(32 * TS)
mingru_scan_sliced_kernel(const float* __restrict__ proj, long long ld, int z_col, int x_col, int g_col, const TB* __restrict__ z_bias,
                          const TB* __restrict__ x_bias, float* __restrict__ state, const int* __restrict__ q_start,
                          const int* __restrict__ state_slot, TO* __restrict__ out, int width)
{
    __shared__ float sa[TS][32], sb[TS][32];
    pdl_enter();
    const int lane = threadIdx.x, ts = threadIdx.y, seq = blockIdx.y;
    const int c = blockIdx.x * 32 + lane;
    const int start = q_start[seq], L = q_start[seq + 1] - start;
    if (L <= 0) return;
    const int per = (L + TS - 1) / TS;
    const int t0 = start + min(ts * per, L), t1 = start + min((ts + 1) * per, L);
    const bool live = c < width;
    const int cc = live ? c : 0;
    const float bz = z_bias != nullptr ? to_f32(z_bias[cc]) : 0.f, bx = x_bias != nullptr ? to_f32(x_bias[cc]) : 0.f;
    float A = 1.f, B = 0.f;
    const float* p = proj + (long long)t0 * ld + cc;
    // four tokens' loads are under way before the first of them is used
    for (int t = t0; t < t1; t += 4, p += 4 * ld) {
        float pz[4], px[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const bool in = t + i < t1;
            pz[i] = in ? p[(long long)i * ld + z_col] : 0.f;
            px[i] = in ? p[(long long)i * ld + x_col] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (t + i >= t1) break;
            const float z = sigmoidf_(pz[i] + bz);
            const float u = px[i] + bx;
            const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
            A *= 1.0f - z;
            B = (1.0f - z) * B + z * cand;
        }
    }
    sa[ts][lane] = A;
    sb[ts][lane] = B;
    __syncthreads();
    float* st = state + (long long)state_slot[seq] * width + cc;
    if (ts == 0) {
        float S = live ? *st : 0.f;
#pragma unroll
        for (int s = 0; s < TS; ++s) {
            const float a = sa[s][lane], b = sb[s][lane];
            sb[s][lane] = S;
            S = a * S + b;
        }
    }
    __syncthreads();
    float S = sb[ts][lane];
    p = proj + (long long)t0 * ld + cc;
    for (int t = t0; t < t1; t += 4, p += 4 * ld) {
        float pz[4], px[4], pg[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const bool in = t + i < t1;
            pz[i] = in ? p[(long long)i * ld + z_col] : 0.f;
            px[i] = in ? p[(long long)i * ld + x_col] : 0.f;
            pg[i] = in ? p[(long long)i * ld + g_col] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (t + i >= t1) break;
            const float z = sigmoidf_(pz[i] + bz);
            const float u = px[i] + bx;
            const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
            S = (1.0f - z) * S + z * cand;
            if (live) out[(long long)(t + i) * width + c] = from_f32<TO>(S * (pg[i] * sigmoidf_(pg[i])));
        }
    }
    if (live && t0 < t1 && t1 == start + L) *st = S;          // the slice that holds the run's last token leaves the state
}

// proj [T, ld] float32 holds the pre-activations of z, of the candidate and of the output gate at the given columns
// (`width` each); biases of z and the candidate or none; state [slots, width]; out [T, width].  `longest`: no request brings
// more tokens than this (runs longer than SCAN_SLICED_FROM take the kernel that is parallel over time).
extern "C" int spy_mingru_scan(const float* proj, long long ld, int z_col, int x_col, int g_col, const void* z_bias, const void* x_bias, int bias_dtype,
                               float* state, const int* q_start, const int* state_slot, int seqs, int longest, void* out, int out_dtype, int width,
                               cudaStream_t stream)
{
    if (seqs <= 0) return 0;
    if (width <= 0 || seqs > 65535) SPY_FAIL("mingru_scan: width %d, %d requests", width, seqs);
    if (z_bias == nullptr && x_bias == nullptr) bias_dtype = SPY_F32;
    SPY_DISPATCH_DTYPE(bias_dtype, TB, {
        SPY_DISPATCH_DTYPE(out_dtype, TO, {
            if (longest > SCAN_SLICED_FROM)
                spy_launch(mingru_scan_sliced_kernel<TB, TO, 32>, dim3((width + 31) / 32, seqs), dim3(32, 32), 0, stream, proj, ld, z_col, x_col, g_col,
                           (const TB*)z_bias, (const TB*)x_bias, state, q_start, state_slot, (TO*)out, width);
            else
                spy_launch(mingru_scan_kernel<TB, TO>, dim3((width + 127) / 128, seqs), dim3(128), 0, stream, proj, ld, z_col, x_col, g_col,
                           (const TB*)z_bias, (const TB*)x_bias, state, q_start, state_slot, (TO*)out, width);
        })
    })
    SPY_CHECK_LAUNCH("mingru_scan");
    return 0;
}

constexpr float LOG2E = 1.4426950408889634f;
constexpr int SS_PER_THREAD = 16;
// 2^v by the special-function unit (two units in the last place at most): the decays of the selective scan, of which a long
// run needs one for every token, channel and state, twice
__device__ __forceinline__ float fast_exp2(float v)
{
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}

// four consecutive entries of a token's B or C row, as one 16-byte load where the row allows it
__device__ __forceinline__ float4 row_quad(const float* __restrict__ p, int n, int n_state, bool vec)
{
    if (vec) return __ldg(reinterpret_cast<const float4*>(p + n));
    float4 v;
    v.x = n < n_state ? __ldg(p + n) : 0.f;
    v.y = n + 1 < n_state ? __ldg(p + n + 1) : 0.f;
    v.z = n + 2 < n_state ? __ldg(p + n + 2) : 0.f;
    v.w = n + 3 < n_state ? __ldg(p + n + 3) : 0.f;
    return v;
}
      // states a thread keeps in registers; a channel's states are dealt out over `lanes` threads

template <typename TX, typename TW, typename TO>
__global__ void selective_scan_kernel(const TX* __restrict__ x, const float* __restrict__ dt_pre, const TW* __restrict__ dt_bias,
                                      const float* __restrict__ proj, long long proj_ld, int b_col, int c_col, const float* __restrict__ z,
                                      long long z_ld, const TW* __restrict__ a_log, const TW* __restrict__ d_skip, float* __restrict__ state,
                                      const int* __restrict__ q_start, const int* __restrict__ state_slot, TO* __restrict__ out, int inner, int n_state,
                                      int lanes)
{
    pdl_enter();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int c = idx / lanes, part = idx % lanes, seq = blockIdx.y;
    const int start = q_start[seq], end = q_start[seq + 1];
    const bool live = c < inner && start < end;          // threads past the last channel still take part in the shuffles
    const bool quads = lanes == 1 && n_state % 4 == 0 && ((proj_ld | b_col | c_col) & 3) == 0;      // B and C rows by 16-byte loads
    const int cc = live ? c : 0;
    float A[SS_PER_THREAD], S[SS_PER_THREAD];
    float* st = state + ((long long)state_slot[seq] * inner + cc) * n_state;
#pragma unroll
    for (int j = 0; j < SS_PER_THREAD; ++j) {
        const int n = part + j * lanes;
        const bool ok = live && n < n_state;
        A[j] = ok ? -expf(to_f32(a_log[(long long)cc * n_state + n])) * LOG2E : 0.f;        // decays as powers of two
        S[j] = ok && !quads ? st[n] : 0.f;
    }
    if (quads && live) {                                     // the thread's states are a run of whole quads
#pragma unroll
        for (int j = 0; j < SS_PER_THREAD; j += 4) {
            if (j >= n_state) break;
            const float4 v = *reinterpret_cast<const float4*>(st + j);
            S[j] = v.x; S[j + 1] = v.y; S[j + 2] = v.z; S[j + 3] = v.w;
        }
    }
    const float bias = live ? to_f32(dt_bias[cc]) : 0.f, D = live ? to_f32(d_skip[cc]) : 0.f;
    for (int t = start; t < end; ++t) {
        const float pre = live ? dt_pre[(long long)t * inner + cc] + bias : 0.f;
        const float dt = pre > 20.f ? pre : log1pf(expf(pre));
        const float xv = live ? to_f32(x[(long long)t * inner + cc]) : 0.f;
        const float dx = dt * xv;
        const float* B = proj + (long long)t * proj_ld + b_col;
        const float* C = proj + (long long)t * proj_ld + c_col;
        float y = 0.f;
        if (lanes == 1) {
#pragma unroll
            for (int j = 0; j < SS_PER_THREAD; j += 4) {
                if (j >= n_state) break;
                const float4 b = row_quad(B, j, n_state, quads), cq = row_quad(C, j, n_state, quads);
                S[j] = fast_exp2(dt * A[j]) * S[j] + dx * b.x;
                S[j + 1] = fast_exp2(dt * A[j + 1]) * S[j + 1] + dx * b.y;
                S[j + 2] = fast_exp2(dt * A[j + 2]) * S[j + 2] + dx * b.z;
                S[j + 3] = fast_exp2(dt * A[j + 3]) * S[j + 3] + dx * b.w;
                y = fmaf(S[j], cq.x, fmaf(S[j + 1], cq.y, fmaf(S[j + 2], cq.z, fmaf(S[j + 3], cq.w, y))));
            }
        } else {
#pragma unroll
            for (int j = 0; j < SS_PER_THREAD; ++j) {
                const int n = part + j * lanes;
                if (n < n_state) {
                    S[j] = fast_exp2(dt * A[j]) * S[j] + dx * __ldg(B + n);
                    y = fmaf(S[j], __ldg(C + n), y);
                }
            }
        }
        for (int o = lanes >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
        if (live && part == 0) {
            y = fmaf(D, xv, y);
            const float zv = z[(long long)t * z_ld + cc];
            out[(long long)t * inner + cc] = from_f32<TO>(y * (zv * sigmoidf_(zv)));
        }
    }
    if (live && quads) {
#pragma unroll
        for (int j = 0; j < SS_PER_THREAD; j += 4) {
            if (j >= n_state) break;
            *reinterpret_cast<float4*>(st + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
        }
    } else if (live) {
#pragma unroll
        for (int j = 0; j < SS_PER_THREAD; ++j) {
            const int n = part + j * lanes;
            if (n < n_state) st[n] = S[j];
        }
    }
}

// The selective scan over long runs, parallel over time in the same way: within a slice the states' decay is
// exp(A[c, n] * sum of dt), so a slice folds into (sum of dt, the states it ends on from zero); the slices are chained from the
// request's states, and each slice then walks its tokens again from the states it starts on.  Blocks of 32 channel-lanes x TS
// slices; the chain over slices is done by TS threads per channel-lane, one for every TS-th state of the lane.
template <typename TX, typename TW, typename TO, int TS>
__global__ void __launch_bounds__(32 * TS)
selective_scan_sliced_kernel(const TX* __restrict__ x, const float* __restrict__ dt_pre, const TW* __restrict__ dt_bias,
                             const float* __restrict__ proj, long long proj_ld, int b_col, int c_col, const float* __restrict__ z,
                             long long z_ld, const TW* __restrict__ a_log, const TW* __restrict__ d_skip, float* __restrict__ state,
                             const int* __restrict__ q_start, const int* __restrict__ state_slot, TO* __restrict__ out, int inner, int n_state,
                             int lanes)
{
    __shared__ float s_end[TS][32][SS_PER_THREAD + 1];
    __shared__ float s_dt[TS][32];
    __shared__ __align__(16) float s_bc[TS][32];            // a slice's current token: B in the first half, C in the second
    pdl_enter();
    const int lx = threadIdx.x, ts = threadIdx.y, seq = blockIdx.y;
    const int idx = blockIdx.x * 32 + lx;
    const int c = idx / lanes, part = idx % lanes;
    const int start = q_start[seq], L = q_start[seq + 1] - start;
    if (L <= 0) return;
    const int per = (L + TS - 1) / TS;
    const int t0 = start + min(ts * per, L), t1 = start + min((ts + 1) * per, L);
    const bool live = c < inner;
    const int cc = live ? c : 0;
    float A[SS_PER_THREAD], S[SS_PER_THREAD];
    float* st = state + ((long long)state_slot[seq] * inner + cc) * n_state;
#pragma unroll
    for (int j = 0; j < SS_PER_THREAD; ++j) {
        const int n = part + j * lanes;
        A[j] = (live && n < n_state) ? -expf(to_f32(a_log[(long long)cc * n_state + n])) * LOG2E : 0.f;       // decays as powers of two
        S[j] = 0.f;
    }
    const float bias = live ? to_f32(dt_bias[cc]) : 0.f, D = live ? to_f32(d_skip[cc]) : 0.f;
    float sum_dt = 0.f;
    // what the next step reads, fetched while the current one is computed; with one thread a channel the token's B and C rows
    // (zeros past the last state) come in by one load of the warp and go round through shared memory
    float pre_n = 0.f, x_n = 0.f, z_n = 0.f, bc_n = 0.f;
    auto fetch = [&](int t, bool gate) {
        if (t >= t1) return;
        pre_n = live ? dt_pre[(long long)t * inner + cc] : 0.f;
        x_n = live ? to_f32(x[(long long)t * inner + cc]) : 0.f;
        if (gate) z_n = live ? z[(long long)t * z_ld + cc] : 0.f;
        if (lanes == 1) bc_n = (lx & 15) < n_state ? __ldg(proj + (long long)t * proj_ld + (lx < 16 ? b_col : c_col) + (lx & 15)) : 0.f;
    };
    fetch(t0, false);
    for (int t = t0; t < t1; ++t) {
        const float pre = pre_n + bias, xv = x_n, bc = bc_n;
        fetch(t + 1, false);
        const float dt = pre > 20.f ? pre : log1pf(expf(pre));
        const float dx = dt * xv;
        sum_dt += dt;
        if (lanes == 1) {
            __syncwarp();
            s_bc[ts][lx] = bc;
            __syncwarp();
#pragma unroll
            for (int j = 0; j < SS_PER_THREAD; j += 4) {
                if (j >= n_state) break;
                const float4 b = *reinterpret_cast<const float4*>(&s_bc[ts][j]);
                S[j] = fast_exp2(dt * A[j]) * S[j] + dx * b.x;
                S[j + 1] = fast_exp2(dt * A[j + 1]) * S[j + 1] + dx * b.y;
                S[j + 2] = fast_exp2(dt * A[j + 2]) * S[j + 2] + dx * b.z;
                S[j + 3] = fast_exp2(dt * A[j + 3]) * S[j + 3] + dx * b.w;
            }
        } else {
            const float* B = proj + (long long)t * proj_ld + b_col;
#pragma unroll
            for (int j = 0; j < SS_PER_THREAD; ++j) {
                const int n = part + j * lanes;
                if (n < n_state) S[j] = fast_exp2(dt * A[j]) * S[j] + dx * __ldg(B + n);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < SS_PER_THREAD; ++j) s_end[ts][lx][j] = S[j];
    s_dt[ts][lx] = sum_dt;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < SS_PER_THREAD; ++j) {
        if (j % TS != ts) continue;                              // this thread chains state j of its channel-lane through the slices
        const int n = part + j * lanes;
        float h = (live && n < n_state) ? st[n] : 0.f;
        for (int s = 0; s < TS; ++s) {
            const float from_zero = s_end[s][lx][j];
            s_end[s][lx][j] = h;
            h = fast_exp2(A[j] * s_dt[s][lx]) * h + from_zero;
        }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < SS_PER_THREAD; ++j) S[j] = s_end[ts][lx][j];
    fetch(t0, true);
    for (int t = t0; t < t1; ++t) {
        const float pre = pre_n + bias, xv = x_n, zv = z_n, bc = bc_n;
        fetch(t + 1, true);
        const float dt = pre > 20.f ? pre : log1pf(expf(pre));
        const float dx = dt * xv;
        float y = 0.f;
        if (lanes == 1) {
            __syncwarp();
            s_bc[ts][lx] = bc;
            __syncwarp();
#pragma unroll
            for (int j = 0; j < SS_PER_THREAD; j += 4) {
                if (j >= n_state) break;
                const float4 b = *reinterpret_cast<const float4*>(&s_bc[ts][j]), cq = *reinterpret_cast<const float4*>(&s_bc[ts][16 + j]);
                S[j] = fast_exp2(dt * A[j]) * S[j] + dx * b.x;
                S[j + 1] = fast_exp2(dt * A[j + 1]) * S[j + 1] + dx * b.y;
                S[j + 2] = fast_exp2(dt * A[j + 2]) * S[j + 2] + dx * b.z;
                S[j + 3] = fast_exp2(dt * A[j + 3]) * S[j + 3] + dx * b.w;
                y = fmaf(S[j], cq.x, fmaf(S[j + 1], cq.y, fmaf(S[j + 2], cq.z, fmaf(S[j + 3], cq.w, y))));
            }
        } else {
            const float* B = proj + (long long)t * proj_ld + b_col;
            const float* C = proj + (long long)t * proj_ld + c_col;
#pragma unroll
            for (int j = 0; j < SS_PER_THREAD; ++j) {
                const int n = part + j * lanes;
                if (n < n_state) {
                    S[j] = fast_exp2(dt * A[j]) * S[j] + dx * __ldg(B + n);
                    y = fmaf(S[j], __ldg(C + n), y);
                }
            }
            for (int o = lanes >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
        }
        if (live && part == 0) {
            y = fmaf(D, xv, y);
            out[(long long)t * inner + cc] = from_f32<TO>(y * (zv * sigmoidf_(zv)));
        }
    }
    if (live && t0 < t1 && t1 == start + L) {
#pragma unroll
        for (int j = 0; j < SS_PER_THREAD; ++j) {
            const int n = part + j * lanes;
            if (n < n_state) st[n] = S[j];
        }
    }
}

// x [T, inner] (after its convolution and activation), dt_pre [T, inner] float32 (the step size before its bias and softplus),
// proj [T, proj_ld] float32 with B at b_col and C at c_col (n_state each), z [T, z_ld] float32 (first `inner` columns from the
// pointer), a_log [inner, n_state], d_skip [inner], dt_bias [inner] of one type; state [slots, inner, n_state]; out [T, inner].
// `longest` as for mingru_scan.
extern "C" int spy_selective_scan(const void* x, int x_dtype, const float* dt_pre, const void* dt_bias, const float* proj, long long proj_ld, int b_col,
                                  int c_col, const float* z, long long z_ld, const void* a_log, const void* d_skip, int weight_dtype, float* state,
                                  const int* q_start, const int* state_slot, int seqs, int longest, void* out, int out_dtype, int inner, int n_state,
                                  cudaStream_t stream)
{
    if (seqs <= 0) return 0;
    if (inner <= 0 || n_state <= 0 || n_state > 32 * SS_PER_THREAD || seqs > 65535)
        SPY_FAIL("selective_scan: %d channels of %d states (at most %d), %d requests", inner, n_state, 32 * SS_PER_THREAD, seqs);
    int lanes = 1;
    while (lanes * SS_PER_THREAD < n_state) lanes *= 2;
    const long long threads = (long long)inner * lanes;
    SPY_DISPATCH_DTYPE(x_dtype, TX, {
        SPY_DISPATCH_DTYPE(weight_dtype, TW, {
            SPY_DISPATCH_DTYPE(out_dtype, TO, {
                if (longest > SCAN_SLICED_FROM)
                    spy_launch(selective_scan_sliced_kernel<TX, TW, TO, 16>, dim3((unsigned)((threads + 31) / 32), seqs), dim3(32, 16), 0, stream,
                               (const TX*)x, dt_pre, (const TW*)dt_bias, proj, proj_ld, b_col, c_col, z, z_ld, (const TW*)a_log, (const TW*)d_skip, state,
                               q_start, state_slot, (TO*)out, inner, n_state, lanes);
                else
                    spy_launch(selective_scan_kernel<TX, TW, TO>, dim3((unsigned)((threads + 127) / 128), seqs), dim3(128), 0, stream, (const TX*)x, dt_pre,
                               (const TW*)dt_bias, proj, proj_ld, b_col, c_col, z, z_ld, (const TW*)a_log, (const TW*)d_skip, state, q_start, state_slot,
                               (TO*)out, inner, n_state, lanes);
            })
        })
    })
    SPY_CHECK_LAUNCH("selective_scan");
    return 0;
}
