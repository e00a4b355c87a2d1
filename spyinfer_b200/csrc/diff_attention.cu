// The steps around the attention kernel of differential attention: every head has two score maps over the same values,
// and the second map's result is subtracted from the first's, `lambda` times.
//
// The two maps of a head run as two query heads of the ordinary attention kernels over ONE key/value head whose key row is
// [key of map 1 | key of map 2]: the query of map m is stored with zeros in the other map's columns, so that its product
// with the key row is the product with its own map's key.  With `heads` heads over `kv_heads` key/value heads, query/key
// size `dim` a map and value size `vdim`, the attention kernels see 2 * heads query heads over kv_heads key/value heads of
// row width `hd` >= max(2 * dim, vdim) (what lies beyond a row's content is zero).
//
// diff_qkv_store: the projection's rows (q | k | v at given columns, plus an optional bias) -> per map RMS norm over dim
//   with a weight shared by all heads and maps, rotation of the pairs (2i, 2i + 1) of each map's first elements by a
//   (cos, sin) table, queries to q_out [T, 2 heads, hd], key rows and values to the pages through the block table.
// diff_combine: o = a1 - lambda a2 per head, divided by its root mean square over vdim (no weight), times `post`, times
//   sigmoid(gate).  All arithmetic in 32-bit.
#include "common.cuh"

SPY_MODULE(spy_diff_attention)

template <typename TP, typename TB, typename TW, typename TQ, typename TC>
__global__ void diff_qkv_store_kernel(const TP* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, const TB* __restrict__ bias,
                                      const TW* __restrict__ q_weight, const TW* __restrict__ k_weight, float eps, const float* __restrict__ rope,
                                      int rot_half, int table_rows, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                      TQ* __restrict__ q_out, const int* __restrict__ block_table, int table_width, TC* __restrict__ pages,
                                      int page_size, int num_pages, int heads, int kv_heads, int dim, int vdim, int hd, int* status)
{
    pdl_enter();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int pos = positions[t];
    bool pos_ok = true;
    if (rot_half > 0 && (pos < 0 || pos >= table_rows)) {
        if (threadIdx.x == 0) report_status(status, SPY_STATUS_BAD_POSITION, t);
        pos_ok = false;
    }
    // where this token's key row and value row go
    long long k_base = -1, v_base = -1;
    {
        const int seq = seq_of_token[t];
        const int lp = pos >= 0 ? pos / page_size : -1;
        const int page = (lp >= 0 && lp < table_width) ? block_table[(long long)seq * table_width + lp] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) report_status(status, SPY_STATUS_BAD_PAGE, t);
        } else {
            k_base = (((long long)page * 2 + 0) * kv_heads * page_size + pos % page_size) * hd;
            v_base = (((long long)page * 2 + 1) * kv_heads * page_size + pos % page_size) * hd;
        }
    }
    const TP* row = proj + (long long)t * ld;
    const int q_units = 2 * heads, k_units = 2 * kv_heads, units = q_units + k_units + kv_heads;
    const int pairs = (dim + 1) / 2;
    for (int u = warp; u < units; u += nwarps) {
        if (u >= q_units + k_units) {
            // a value head: copied, the rest of the row zero
            const int g = u - q_units - k_units;
            if (v_base < 0) continue;
            TC* dst = pages + v_base + (long long)g * page_size * hd;
            for (int e = lane; e < hd; e += 32) {
                float v = 0.f;
                if (e < vdim) {
                    const int col = v_col + g * vdim + e;
                    v = to_f32(row[col]) + (bias != nullptr ? to_f32(bias[col]) : 0.f);
                }
                dst[e] = from_f32<TC>(v);
            }
            continue;
        }
        const bool is_q = u < q_units;
        const int head = (is_q ? u : u - q_units) / 2, map = (is_q ? u : u - q_units) % 2;
        const int col0 = (is_q ? q_col : k_col) + (head * 2 + map) * dim;
        const TW* w = is_q ? q_weight : k_weight;
        // unit root mean square over the map's dim elements
        float ss = 0.f;
        for (int e = lane; e < dim; e += 32) {
            const float v = to_f32(row[col0 + e]) + (bias != nullptr ? to_f32(bias[col0 + e]) : 0.f);
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        const float rstd = 1.0f / sqrtf(ss / (float)dim + eps);
        if (is_q) {
            TQ* dst = q_out + ((long long)t * q_units + u) * hd;
            for (int e = lane; e < hd; e += 32)
                if (e < map * dim || e >= map * dim + dim) dst[e] = from_f32<TQ>(0.f);
        } else if (k_base >= 0 && map == 0) {
            TC* dst = pages + k_base + (long long)head * page_size * hd;
            for (int e = 2 * dim + lane; e < hd; e += 32) dst[e] = from_f32<TC>(0.f);
        }
        for (int p = lane; p < pairs; p += 32) {
            const int e0 = 2 * p, e1 = 2 * p + 1;
            float a = (to_f32(row[col0 + e0]) + (bias != nullptr ? to_f32(bias[col0 + e0]) : 0.f)) * rstd * to_f32(w[e0]);
            float b = 0.f;
            if (e1 < dim) b = (to_f32(row[col0 + e1]) + (bias != nullptr ? to_f32(bias[col0 + e1]) : 0.f)) * rstd * to_f32(w[e1]);
            if (p < rot_half && pos_ok) {
                const float c = rope[((long long)pos * rot_half + p) * 2], s = rope[((long long)pos * rot_half + p) * 2 + 1];
                const float ra = a * c - b * s, rb = b * c + a * s;
                a = ra;
                b = rb;
            }
            if (is_q) {
                TQ* dst = q_out + ((long long)t * q_units + u) * hd + map * dim;
                dst[e0] = from_f32<TQ>(a);
                if (e1 < dim) dst[e1] = from_f32<TQ>(b);
            } else if (k_base >= 0) {
                TC* dst = pages + k_base + (long long)head * page_size * hd + map * dim;
                dst[e0] = from_f32<TC>(a);
                if (e1 < dim) dst[e1] = from_f32<TC>(b);
            }
        }
    }
}

extern "C" int spy_diff_qkv_store(const void* proj, int proj_dtype, long long ld, int q_col, int k_col, int v_col, const void* bias, int bias_dtype,
                                  const void* q_weight, const void* k_weight, int weight_dtype, float eps, const float* rope, int rot_half,
                                  int table_rows, const int* positions, const int* seq_of_token, void* q_out, int q_dtype, const int* block_table,
                                  int table_width, void* pages, int cache_dtype, int page_size, int num_pages, int tokens, int heads, int kv_heads,
                                  int dim, int vdim, int hd, int* status, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || hd < 2 * dim || hd < vdim)
        SPY_FAIL("diff_qkv_store: %d heads, %d key/value heads, dim %d, vdim %d do not fit rows of %d", heads, kv_heads, dim, vdim, hd);
    if (2 * rot_half > dim) SPY_FAIL("diff_qkv_store: %d rotated pairs do not fit a map of %d elements", rot_half, dim);
    if (page_size <= 0 || num_pages <= 0 || table_width <= 0) SPY_FAIL("diff_qkv_store: page_size, num_pages and table_width must be positive");
    if (bias == nullptr) bias_dtype = SPY_F32;
    if (proj_dtype != q_dtype && proj_dtype != SPY_F32) SPY_FAIL("diff_qkv_store: the projection is float32 or has the queries' type");
    if (q_dtype != cache_dtype) SPY_FAIL("diff_qkv_store: queries and cache have one type");
#define SPY_DQS(TP, TB, TW, TQ)                                                                                                          \
    spy_launch(diff_qkv_store_kernel<TP, TB, TW, TQ, TQ>, dim3(tokens), dim3(128), 0, stream, (const TP*)proj, ld, q_col, k_col, v_col,   \
               (const TB*)bias, (const TW*)q_weight, (const TW*)k_weight, eps, rope, rot_half, table_rows, positions, seq_of_token,       \
               (TQ*)q_out, block_table, table_width, (TQ*)pages, page_size, num_pages, heads, kv_heads, dim, vdim, hd, status)
    SPY_DISPATCH_DTYPE(bias_dtype, TB, {
        SPY_DISPATCH_DTYPE(weight_dtype, TW, {
            if (q_dtype == SPY_F32) SPY_DQS(float, TB, TW, float);
            else if (proj_dtype == SPY_F32) SPY_DQS(float, TB, TW, bf16);
            else SPY_DQS(bf16, TB, TW, bf16);
        })
    })
#undef SPY_DQS
    SPY_CHECK_LAUNCH("diff_qkv_store");
    return 0;
}

template <typename TA, typename TG, typename TO>
__global__ void diff_combine_kernel(const TA* __restrict__ attn, int hd, const TG* __restrict__ gate, long long gate_ld, int gate_col,
                                    TO* __restrict__ out, int tokens, int heads, int vdim, float lambda, float post, float eps)
{
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)tokens * heads) return;
    const long long t = unit / heads;
    const int h = (int)(unit % heads);
    const TA* a1 = attn + (t * 2 * heads + 2 * h) * hd;
    const TA* a2 = a1 + hd;
    float ss = 0.f;
    for (int e = lane; e < vdim; e += 32) {
        const float o = to_f32(a1[e]) - lambda * to_f32(a2[e]);
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float mul = post / sqrtf(ss / (float)vdim + eps);
    for (int e = lane; e < vdim; e += 32) {
        float o = (to_f32(a1[e]) - lambda * to_f32(a2[e])) * mul;
        if (gate != nullptr) o = o / (1.0f + expf(-to_f32(gate[t * gate_ld + gate_col + h * vdim + e])));
        out[(t * heads + h) * vdim + e] = from_f32<TO>(o);
    }
}

// attn [T, 2 heads, hd] (map 1 and map 2 of each head side by side, the first vdim elements of each row), gate [T, gate_ld]
// read from column gate_col (or none), out [T, heads * vdim].
extern "C" int spy_diff_combine(const void* attn, int attn_dtype, int hd, const void* gate, int gate_dtype, long long gate_ld, int gate_col, void* out,
                                int out_dtype, int tokens, int heads, int vdim, float lambda, float post, float eps, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (heads <= 0 || vdim <= 0 || hd < vdim) SPY_FAIL("diff_combine: %d heads of %d values do not fit rows of %d", heads, vdim, hd);
    if (gate == nullptr) gate_dtype = SPY_F32;
    const long long units = (long long)tokens * heads;
    const int per_block = 4;
    SPY_DISPATCH_DTYPE(attn_dtype, TA, {
        SPY_DISPATCH_DTYPE(gate_dtype, TG, {
            SPY_DISPATCH_DTYPE(out_dtype, TO, {
                spy_launch(diff_combine_kernel<TA, TG, TO>, dim3((unsigned)((units + per_block - 1) / per_block)), dim3(32 * per_block), 0, stream,
                           (const TA*)attn, hd, (const TG*)gate, gate_ld, gate_col, (TO*)out, tokens, heads, vdim, lambda, post, eps);
            })
        })
    })
    SPY_CHECK_LAUNCH("diff_combine");
    return 0;
}
