// The steps around the attention kernels for attention whose queries and keys are normed over the whole projection,
// whose values have unit root mean square, whose heads have a temperature, and whose softmax has a sink.
//
// sink_qkv_store: one block a token.  From the projection's row (q | k | v at given columns, 32-bit or the activations' type):
//   q = q / sqrt(mean(q^2 over ALL heads) + eps) * q_weight   (one statistic for the row's heads * dim elements), the same for
//   k over its kv_heads * dim elements; rotation of the pairs (2i, 2i + 1), i < rot_half, of every head by a (cos, sin) table;
//   q times the head's temperature (so that the attention kernels' one scale serves every head); every value head divided by
//   sqrt(mean(v^2 over vdim) + eps), no weight.  Queries go to q_out [T, heads, hd], keys and values through the block table
//   into pages of rows hd >= max(dim, vdim); what lies beyond a row's content is zero.  A layer that reads another layer's
//   keys and values passes no pages and gets its queries only.
// sink_merge: one warp a (token, head).  An attention kernel has done the keys of the window and left its normalised result
//   and the logarithm of its sum of exponentials; this adds what the window's kernel does not know: the keys of the
//   sequence's first `keep_first` positions that lie before the window, and the sink (a key of score 0 without a value, which
//   adds one to the denominator).
// All arithmetic in 32-bit.
#include "common.cuh"

SPY_MODULE(spy_sink_attention)

// four consecutive elements, 16-byte (float) or 8-byte (bfloat16) accesses
__device__ __forceinline__ void load4(const float* p, float (&v)[4])
{
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
__device__ __forceinline__ void load4(const bf16* p, float (&v)[4])
{
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x), b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4])
{
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 x;
    x.x = *reinterpret_cast<uint32_t*>(&a);
    x.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = x;
}

// VEC: dim, vdim, hd, the columns and the row pitch are multiples of 4, rot_half is even and every array is aligned for
// 4-element accesses: a thread takes two neighbouring pairs at a time.
template <typename TP, typename TW, typename TQ, bool VEC>
__global__ void __launch_bounds__(256)
sink_qkv_store_kernel(const TP* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, const TW* __restrict__ q_weight,
                      const TW* __restrict__ k_weight, const TW* __restrict__ temp, float eps, const float* __restrict__ rope, int rot_half,
                      int table_rows, const int* __restrict__ positions, const int* __restrict__ seq_of_token, TQ* __restrict__ q_out,
                      const int* __restrict__ block_table, int table_width, TQ* __restrict__ pages, int page_size, int num_pages, int heads,
                      int kv_heads, int dim, int vdim, int hd, int* status)
{
    __shared__ float scratch[33];
    pdl_enter();
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int pos = positions[t];
    const bool stores = pages != nullptr;
    bool pos_ok = true;
    if (rot_half > 0 && (pos < 0 || pos >= table_rows)) {
        if (tid == 0) report_status(status, SPY_STATUS_BAD_POSITION, t);
        pos_ok = false;
    }
    long long k_base = -1, v_base = -1;
    if (stores) {
        const int seq = seq_of_token[t];
        const int lp = pos >= 0 ? pos / page_size : -1;
        const int page = (lp >= 0 && lp < table_width) ? block_table[(long long)seq * table_width + lp] : -1;
        if (page < 0 || page >= num_pages) {
            if (tid == 0) report_status(status, SPY_STATUS_BAD_PAGE, t);
        } else {
            k_base = (((long long)page * 2 + 0) * kv_heads * page_size + pos % page_size) * hd;
            v_base = (((long long)page * 2 + 1) * kv_heads * page_size + pos % page_size) * hd;
        }
    }
    const TP* row = proj + (long long)t * ld;
    const int nq = heads * dim, nk = kv_heads * dim;
    // one root mean square for all of q, one for all of k
    float sq = 0.f, sk = 0.f;
    if constexpr (VEC) {
        for (int e = tid * 4; e < nq; e += blockDim.x * 4) {
            float v[4];
            load4(row + q_col + e, v);
            sq += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        }
        if (stores)
            for (int e = tid * 4; e < nk; e += blockDim.x * 4) {
                float v[4];
                load4(row + k_col + e, v);
                sk += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
            }
    } else {
        for (int e = tid; e < nq; e += blockDim.x) {
            const float v = to_f32(row[q_col + e]);
            sq = fmaf(v, v, sq);
        }
        if (stores)
            for (int e = tid; e < nk; e += blockDim.x) {
                const float v = to_f32(row[k_col + e]);
                sk = fmaf(v, v, sk);
            }
    }
    sq = block_sum(sq, scratch);
    if (stores) sk = block_sum(sk, scratch);
    const float rq = 1.0f / sqrtf(sq / (float)nq + eps), rk = 1.0f / sqrtf(sk / (float)max(nk, 1) + eps);
    if constexpr (VEC) {
        // queries, then keys, then values: a thread takes four neighbouring elements (two pairs) of a head's row
        const int quads = hd / 4, q_items = heads * quads, k_items = stores ? kv_heads * quads : 0;
        for (int it = tid; it < q_items + k_items; it += blockDim.x) {
            const bool is_q = it < q_items;
            const int idx = is_q ? it : it - q_items;
            const int head = idx / quads, e0 = 4 * (idx - head * quads);
            float o[4] = {0.f, 0.f, 0.f, 0.f};
            if (e0 < dim) {
                float x[4], w[4];
                load4(row + (is_q ? q_col : k_col) + head * dim + e0, x);
                load4((is_q ? q_weight : k_weight) + head * dim + e0, w);
                const float r = is_q ? rq : rk;
#pragma unroll
                for (int i = 0; i < 4; ++i) o[i] = x[i] * r * w[i];
                const int p = e0 / 2;
                if (p < rot_half && pos_ok) {
                    float cs[4];
                    load4(rope + ((long long)pos * rot_half + p) * 2, cs);
                    const float a0 = o[0] * cs[0] - o[1] * cs[1], b0 = o[1] * cs[0] + o[0] * cs[1];
                    const float a1 = o[2] * cs[2] - o[3] * cs[3], b1 = o[3] * cs[2] + o[2] * cs[3];
                    o[0] = a0; o[1] = b0; o[2] = a1; o[3] = b1;
                }
                if (is_q && temp != nullptr) {
                    const float tau = to_f32(temp[head]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[i] *= tau;
                }
            }
            if (is_q) store4(q_out + ((long long)t * heads + head) * hd + e0, o);
            else if (k_base >= 0) store4(pages + k_base + (long long)head * page_size * hd + e0, o);
        }
        if (stores) {
            for (int g = warp; g < kv_heads; g += nwarps) {
                const TP* src = row + v_col + g * vdim;
                float ss = 0.f;
                for (int e = lane * 4; e < vdim; e += 128) {
                    float v[4];
                    load4(src + e, v);
                    ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
                }
                ss = warp_sum(ss);
                const float rv = 1.0f / sqrtf(ss / (float)vdim + eps);
                if (v_base < 0) continue;
                TQ* dst = pages + v_base + (long long)g * page_size * hd;
                for (int e = lane * 4; e < hd; e += 128) {
                    float v[4] = {0.f, 0.f, 0.f, 0.f};
                    if (e < vdim) {
                        load4(src + e, v);
#pragma unroll
                        for (int i = 0; i < 4; ++i) v[i] *= rv;
                    }
                    store4(dst + e, v);
                }
            }
        }
        return;
    }
    const int pairs = (dim + 1) / 2, slots = hd / 2 + (hd & 1);      // pairs of a head's content; pairs of a whole row
    // queries, then keys: a thread takes a pair of neighbouring elements of a head's row
    const int q_items = heads * slots, k_items = stores ? kv_heads * slots : 0;
    for (int it = tid; it < q_items + k_items; it += blockDim.x) {
        const bool is_q = it < q_items;
        const int idx = is_q ? it : it - q_items;
        const int head = idx / slots, p = idx - head * slots;
        const int e0 = 2 * p, e1 = 2 * p + 1;
        float a = 0.f, b = 0.f;
        if (p < pairs) {
            const int col = (is_q ? q_col : k_col) + head * dim;
            const TW* w = (is_q ? q_weight : k_weight) + head * dim;
            const float r = is_q ? rq : rk;
            a = to_f32(row[col + e0]) * r * to_f32(w[e0]);
            if (e1 < dim) b = to_f32(row[col + e1]) * r * to_f32(w[e1]);
            if (p < rot_half && pos_ok) {
                const float c = rope[((long long)pos * rot_half + p) * 2], s = rope[((long long)pos * rot_half + p) * 2 + 1];
                const float ra = a * c - b * s, rb = b * c + a * s;
                a = ra;
                b = rb;
            }
            if (is_q && temp != nullptr) {
                const float tau = to_f32(temp[head]);
                a *= tau;
                b *= tau;
            }
        }
        if (is_q) {
            TQ* dst = q_out + ((long long)t * heads + head) * hd;
            dst[e0] = from_f32<TQ>(a);
            if (e1 < hd) dst[e1] = from_f32<TQ>(b);
        } else if (k_base >= 0) {
            TQ* dst = pages + k_base + (long long)head * page_size * hd;
            dst[e0] = from_f32<TQ>(a);
            if (e1 < hd) dst[e1] = from_f32<TQ>(b);
        }
    }
    // values: a warp a head
    if (stores) {
        for (int g = warp; g < kv_heads; g += nwarps) {
            const TP* src = row + v_col + g * vdim;
            float ss = 0.f;
            for (int e = lane; e < vdim; e += 32) {
                const float v = to_f32(src[e]);
                ss = fmaf(v, v, ss);
            }
            ss = warp_sum(ss);
            const float rv = 1.0f / sqrtf(ss / (float)vdim + eps);
            if (v_base < 0) continue;
            TQ* dst = pages + v_base + (long long)g * page_size * hd;
            for (int e = lane; e < hd; e += 32) dst[e] = from_f32<TQ>(e < vdim ? to_f32(src[e]) * rv : 0.f);
        }
    }
}

// proj [T, ld]; q_weight [heads * dim], k_weight [kv_heads * dim], temp [heads] (null: no temperature) of weight_dtype;
// rope [table_rows, rot_half, 2] float32 (null with rot_half 0); q_out [T, heads * hd]; pages [num_pages][2][kv_heads][page_size][hd]
// of the queries' type, or null with a null block table: queries only.
extern "C" int spy_sink_qkv_store(const void* proj, int proj_dtype, long long ld, int q_col, int k_col, int v_col, const void* q_weight,
                                  const void* k_weight, const void* temp, int weight_dtype, float eps, const float* rope, int rot_half, int table_rows,
                                  const int* positions, const int* seq_of_token, void* q_out, int q_dtype, const int* block_table, int table_width,
                                  void* pages, int page_size, int num_pages, int tokens, int heads, int kv_heads, int dim, int vdim, int hd, int* status,
                                  cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || hd < dim || hd < vdim)
        SPY_FAIL("sink_qkv_store: %d heads, %d key/value heads, dim %d, vdim %d do not fit rows of %d", heads, kv_heads, dim, vdim, hd);
    if (rot_half < 0 || 2 * rot_half > dim || (rot_half > 0 && rope == nullptr)) SPY_FAIL("sink_qkv_store: %d rotated pairs do not fit a head of %d elements", rot_half, dim);
    if (pages != nullptr && (page_size <= 0 || num_pages <= 0 || table_width <= 0 || block_table == nullptr))
        SPY_FAIL("sink_qkv_store: page_size, num_pages and table_width must be positive");
    if (pages != nullptr && k_weight == nullptr) SPY_FAIL("sink_qkv_store: keys are stored and have no norm weight");
    const auto misaligned = [](const void* p, size_t elt) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) % (4 * elt)) != 0; };
    const size_t pe = proj_dtype == SPY_F32 ? 4 : 2, we = weight_dtype == SPY_F32 ? 4 : 2, qe = q_dtype == SPY_F32 ? 4 : 2;
    const bool vec = dim % 4 == 0 && vdim % 4 == 0 && hd % 4 == 0 && q_col % 4 == 0 && k_col % 4 == 0 && v_col % 4 == 0 && ld % 4 == 0 && rot_half % 2 == 0
                     && !misaligned(proj, pe) && !misaligned(q_weight, we) && !misaligned(k_weight, we) && !misaligned(q_out, qe) && !misaligned(pages, qe)
                     && !misaligned(rope, 4);
    const int threads = tokens >= 512 ? 128 : 256;      // many tokens: more blocks an SM; few: the row spread wide
#define SPY_SQS(TP, TW, TQ)                                                                                                                    \
    do {                                                                                                                                        \
        auto kernel = vec ? sink_qkv_store_kernel<TP, TW, TQ, true> : sink_qkv_store_kernel<TP, TW, TQ, false>;                                  \
        spy_launch(kernel, dim3(tokens), dim3(threads), 0, stream, (const TP*)proj, ld, q_col, k_col, v_col, (const TW*)q_weight,                 \
                   (const TW*)k_weight, (const TW*)temp, eps, rope, rot_half, table_rows, positions, seq_of_token, (TQ*)q_out, block_table, table_width, \
                   (TQ*)pages, page_size, num_pages, heads, kv_heads, dim, vdim, hd, status);                                                    \
    } while (0)
    SPY_DISPATCH_DTYPE(proj_dtype, TP, {
        SPY_DISPATCH_DTYPE(weight_dtype, TW, {
            if (q_dtype == SPY_F32) SPY_SQS(TP, TW, float);
            else if (q_dtype == SPY_BF16) SPY_SQS(TP, TW, bf16);
            else SPY_FAIL("sink_qkv_store: unknown dtype code %d", q_dtype);
        })
    })
#undef SPY_SQS
    SPY_CHECK_LAUNCH("sink_qkv_store");
    return 0;
}

// out[t, h, :] holds sum_j p_j v_j over the window's keys with p normalised over them, lse[t, h] = log(sum_j exp(score_j)).
// With K = the kept keys before the window (positions 0 .. min(keep_first, first key of the window) - 1):
//   M = max(lse, 0, max_K score), D = exp(lse - M) + [sink] exp(-M) + sum_K exp(score - M),
//   out = out * exp(lse - M) / D + sum_K exp(score - M) / D * v.
template <typename TQ>
__global__ void sink_merge_kernel(const TQ* __restrict__ q, long long q_ld, TQ* __restrict__ out, const float* __restrict__ lse,
                                  const TQ* __restrict__ pages, const int* __restrict__ block_table, int table_width, int page_size, int num_pages,
                                  int nh, int nkv, int hd, const int* __restrict__ positions, const int* __restrict__ seq_of_token, int tokens,
                                  int window, int keep_first, int sink, float scale, int* status)
{
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)tokens * nh) return;
    const int t = (int)(item / nh), h = (int)(item - (long long)t * nh);
    const int pos = positions[t], seq = seq_of_token[t], kvh = h / (nh / nkv);
    const int kept = min(keep_first, spy_first_key(pos, window));
    if (kept <= 0 && !sink) return;
    const TQ* qr = q + (long long)t * q_ld + (long long)h * hd;
    TQ* orow = out + ((long long)t * nh + h) * hd;
    const float lw = lse[(long long)t * nh + h];
    const int* bt = block_table + (long long)seq * table_width;
    float m = sink ? fmaxf(lw, 0.f) : lw;
    // scores of the kept keys (a handful)
    float acc[8];                        // the row's elements lane, lane + 32, ...: rows of up to 256
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = 0.f;
    float d_extra = 0.f;                 // sum over kept keys of exp(score - m), m being updated as we go
    float m_run = m;
    {
        for (int j = 0; j < kept; ++j) {
            const int lp = j / page_size;
            const int page = lp < table_width ? bt[lp] : -1;
            if (page < 0 || page >= num_pages) {
                if (lane == 0) report_status(status, SPY_STATUS_BAD_PAGE, t);
                continue;
            }
            const TQ* kr = pages + ((((long long)page * 2) * nkv + kvh) * page_size + j % page_size) * hd;
            const TQ* vr = kr + (long long)nkv * page_size * hd;
            float dot = 0.f;
            for (int e = lane; e < hd; e += 32) dot = fmaf(to_f32(qr[e]), to_f32(kr[e]), dot);
            const float s = warp_sum(dot) * scale;
            const float m_new = fmaxf(m_run, s);
            const float alpha = m_run == -INFINITY ? 0.f : expf(m_run - m_new), p = expf(s - m_new);
            d_extra = d_extra * alpha + p;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const int e = lane + 32 * r;
                if (e < hd) acc[r] = fmaf(p, to_f32(vr[e]), acc[r] * alpha);
            }
            m_run = m_new;
        }
    }
    const float ww = lw == -INFINITY ? 0.f : expf(lw - m_run);                 // the window's weight
    const float denom = ww + d_extra + (sink ? expf(-m_run) : 0.f);
    const float inv = denom > 0.f ? 1.0f / denom : 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const int e = lane + 32 * r;
        if (e < hd) orow[e] = from_f32<TQ>((to_f32(orow[e]) * ww + acc[r]) * inv);
    }
}

// The same for rows of 128 (V = 4) or 64 (V = 2) bfloat16 elements: a lane holds V neighbouring elements of the row, up to
// four kept keys are fetched together and their scores reduced side by side.
template <int V>
__device__ __forceinline__ void load_lane(const bf16* p, float (&v)[V])
{
    if constexpr (V == 4) {
        load4(p, v);
    } else {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(p);
        v[0] = __low2float(a); v[1] = __high2float(a);
    }
}
template <int V>
__device__ __forceinline__ void store_lane(bf16* p, const float (&v)[V])
{
    if constexpr (V == 4) {
        store4(p, v);
    } else {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
    }
}

template <int V>
__global__ void sink_merge_rows_kernel(const bf16* __restrict__ q, long long q_ld, bf16* __restrict__ out, const float* __restrict__ lse,
                                       const bf16* __restrict__ pages, const int* __restrict__ block_table, int table_width, int page_size, int num_pages,
                                       int nh, int nkv, const int* __restrict__ positions, const int* __restrict__ seq_of_token, int tokens,
                                       int window, int keep_first, int sink, float scale, int* status, int group)
{
    constexpr int HD = 32 * V, KB = 4;
    pdl_enter();
    // grid: x = token, y = groups of the block's warps over the heads; a warp a (token, head); no division on the way
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (h >= nh) return;
    const int pos = positions[t], kvh = h / group;
    const int kept = min(keep_first, spy_first_key(pos, window));
    if (kept <= 0 && !sink) return;
    bf16* orow = out + ((long long)t * nh + h) * HD + lane * V;
    const float lw = lse[(long long)t * nh + h];
    float ov[V], acc[V];
    load_lane<V>(orow, ov);
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    float m_run = sink ? fmaxf(lw, 0.f) : lw, d_extra = 0.f;
    if (kept > 0) {
        const int* bt = block_table + (long long)seq_of_token[t] * table_width;
        float qv[V];
        load_lane<V>(q + (long long)t * q_ld + (long long)h * HD + lane * V, qv);
        int lp = 0, slot = 0;                                  // the page and the place in it of key j0 + b, stepped along
        for (int j0 = 0; j0 < kept; j0 += KB) {
            float dot[KB], vv[KB][V];
            bool ok[KB];
#pragma unroll
            for (int b = 0; b < KB; ++b) {
                const int j = j0 + b;
                const int page = (j < kept && lp < table_width) ? bt[lp] : -1;
                ok[b] = page >= 0 && page < num_pages;
                dot[b] = 0.f;
                if (j < kept && !ok[b] && lane == 0) report_status(status, SPY_STATUS_BAD_PAGE, t);
                if (ok[b]) {
                    const bf16* kr = pages + ((((long long)page * 2) * nkv + kvh) * page_size + slot) * HD + lane * V;
                    float kv[V];
                    load_lane<V>(kr, kv);
                    load_lane<V>(kr + (long long)nkv * page_size * HD, vv[b]);
#pragma unroll
                    for (int i = 0; i < V; ++i) dot[b] = fmaf(qv[i], kv[i], dot[b]);
                }
                if (++slot == page_size) {
                    slot = 0;
                    ++lp;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int b = 0; b < KB; ++b) dot[b] += __shfl_xor_sync(0xffffffffu, dot[b], o);
#pragma unroll
            for (int b = 0; b < KB; ++b) {
                if (!ok[b]) continue;
                const float s = dot[b] * scale, m_new = fmaxf(m_run, s);
                const float alpha = m_run == -INFINITY ? 0.f : expf(m_run - m_new), p = expf(s - m_new);
                d_extra = d_extra * alpha + p;
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] = fmaf(p, vv[b][i], acc[i] * alpha);
                m_run = m_new;
            }
        }
    }
    const float ww = lw == -INFINITY ? 0.f : expf(lw - m_run);
    const float denom = ww + d_extra + (sink ? expf(-m_run) : 0.f);
    const float inv = denom > 0.f ? 1.0f / denom : 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) ov[i] = (ov[i] * ww + acc[i]) * inv;
    store_lane<V>(orow, ov);
}

// q [T, q_ld] (heads * hd columns read), out [T, nh * hd] rewritten in place, lse [T, nh] float32, pages as above.
extern "C" int spy_sink_merge(const void* q, long long q_ld, void* out, int act_dtype, const float* lse, const void* pages, const int* block_table,
                              int table_width, int page_size, int num_pages, int nh, int nkv, int hd, const int* positions, const int* seq_of_token,
                              int tokens, int window, int keep_first, int sink, float scale, int* status, cudaStream_t stream)
{
    if (tokens <= 0 || (keep_first <= 0 && !sink)) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || hd > 256) SPY_FAIL("sink_merge: %d heads over %d key/value heads of %d (at most 256)", nh, nkv, hd);
    if (keep_first > 0 && window <= 0) SPY_FAIL("sink_merge: kept first keys go with a window");
    if (lse == nullptr) SPY_FAIL("sink_merge: no logarithms of the window's sums");
    const long long items = (long long)tokens * nh;
    const int warps = 8;
    const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(pages)) & 7) == 0 && q_ld % 4 == 0;
    if (act_dtype == SPY_BF16 && aligned && (hd == 128 || hd == 64)) {
        const int per_block = nh < warps ? nh : warps;
        if ((nh + per_block - 1) / per_block > 65535) SPY_FAIL("sink_merge: %d heads exceed the grid", nh);
        const dim3 grid((unsigned)tokens, (unsigned)((nh + per_block - 1) / per_block)), block(per_block * 32);
        if (hd == 128)
            spy_launch(sink_merge_rows_kernel<4>, grid, block, 0, stream, (const bf16*)q, q_ld, (bf16*)out, lse, (const bf16*)pages, block_table, table_width,
                       page_size, num_pages, nh, nkv, positions, seq_of_token, tokens, window, keep_first, sink, scale, status, nh / nkv);
        else
            spy_launch(sink_merge_rows_kernel<2>, grid, block, 0, stream, (const bf16*)q, q_ld, (bf16*)out, lse, (const bf16*)pages, block_table, table_width,
                       page_size, num_pages, nh, nkv, positions, seq_of_token, tokens, window, keep_first, sink, scale, status, nh / nkv);
        SPY_CHECK_LAUNCH("sink_merge");
        return 0;
    }
    SPY_DISPATCH_DTYPE(act_dtype, TQ, {
        spy_launch(sink_merge_kernel<TQ>, dim3((unsigned)((items + warps - 1) / warps)), dim3(warps * 32), 0, stream, (const TQ*)q, q_ld, (TQ*)out, lse,
                   (const TQ*)pages, block_table, table_width, page_size, num_pages, nh, nkv, hd, positions, seq_of_token, tokens, window, keep_first, sink,
                   scale, status);
    })
    SPY_CHECK_LAUNCH("sink_merge");
    return 0;
}
