// Layer norm with a weight and an optional bias, optionally fused with a scaled residual sum and a row gather.
//   v      = x[row] + scale_a * a_w * sum_s a[s][row] + scale_b * sum_s b[s][row]    32-bit sums, parts in their order
//   x[row] = v                                             when write_back (the residual stream)
//   out    = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w (+ bias)          32-bit statistics, two passes
// a_w (null, or [len] of the weight's type) multiplies the first result element by element along the row (a layer scale);
// a_bias (null, or [len] float32) is added to the first result ahead of that: x += scale_a * a_w * (sum_s a[s] + a_bias), the
// bias of the projection that made the result.  a_rows (null, or [*, len] of the output's type) with a_row_w ([*] float32): a second
// term of the first result with one weight a row, x += scale_a * a_w * (sum_s a[s] + a_bias + a_row_w[row] * a_rows[row]), what the
// identity experts of a mixture contribute (their summed weight times the feed-forward's input).
// a and b are null, one array [*, len], or stacks of split-K partial products (splits arrays, split_stride elements
// apart); two of them because a layer whose mixer is two mixers side by side hands over two results with a weight each.
// With center == 0 the mean is not removed (an RMS norm with the same fused sums).
#include "common.cuh"

SPY_MODULE(spy_layernorm)

template <typename T> struct Quad;
template <> struct Quad<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4])
    {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Quad<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4])
    {
        const uint2 x = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x), b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[4])
    {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 x;
        x.x = *reinterpret_cast<uint32_t*>(&a);
        x.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = x;
    }
};

// VEC: the row length is a multiple of 4 and every array is 16-byte aligned: four elements a load.
// REG > 0 (with VEC): the row is exactly REG quads a thread (len == 4 * REG * blockDim.x) and stays in registers between the passes,
// with all of a thread's loads under way together; REG == 0: any length, the row kept in shared memory.  The sums are formed in
// the same order either way.
template <typename TX, typename TD, typename TW, typename TO, bool VEC, int REG>
__global__ void __launch_bounds__(1024)
layernorm_kernel(TX* x, const TD* __restrict__ a, int a_splits, long long a_stride, float a_scale, const TD* __restrict__ b, int b_splits,
                 long long b_stride, float b_scale, const int* __restrict__ rows, const TW* __restrict__ w, TO* __restrict__ out, int len, float eps,
                 int write_back, int center, const TW* __restrict__ bias, const TW* __restrict__ a_w, const float* __restrict__ a_bias,
                 const TO* __restrict__ a_rows, const float* __restrict__ a_row_w)
{
    extern __shared__ __align__(16) float row_buf[];  // len floats, then 33 of scratch
    pdl_enter();
    float* scratch = row_buf + len;
    const int src_row = rows ? rows[blockIdx.x] : blockIdx.x;
    TX* xr = x + (size_t)src_row * len;
    const TD* ar = a ? a + (size_t)src_row * len : nullptr;
    const TD* br = b ? b + (size_t)src_row * len : nullptr;
    TO* orow = out + (size_t)blockIdx.x * len;
    constexpr int E = VEC ? 4 : 1;
    float sum = 0.f;
    // the sum of everything that goes into the stream at elements i .. i + E - 1 (stored back when asked for)
    const auto gather = [&](int i, float (&v)[4]) {
        float d[4], p[4];
        if constexpr (VEC) Quad<TX>::load(xr + i, v); else v[0] = to_f32(xr[i]);
        if (ar) {
#pragma unroll
            for (int e = 0; e < E; ++e) d[e] = 0.f;
            for (int s = 0; s < a_splits; ++s) {
                if constexpr (VEC) Quad<TD>::load(ar + (size_t)s * a_stride + i, p); else p[0] = to_f32(ar[(size_t)s * a_stride + i]);
#pragma unroll
                for (int e = 0; e < E; ++e) d[e] += p[e];
            }
            if (a_rows) {
                const float rw = a_row_w[src_row];
                float xr4[4];
                if constexpr (VEC) Quad<TO>::load(a_rows + (size_t)src_row * len + i, xr4); else xr4[0] = to_f32(a_rows[(size_t)src_row * len + i]);
#pragma unroll
                for (int e = 0; e < E; ++e) d[e] = fmaf(rw, xr4[e], d[e]);
            }
            if (a_bias) {
                float ab[4];
                if constexpr (VEC) Quad<float>::load(a_bias + i, ab); else ab[0] = a_bias[i];
#pragma unroll
                for (int e = 0; e < E; ++e) d[e] += ab[e];
            }
            if (a_w) {
                float aw[4];
                if constexpr (VEC) Quad<TW>::load(a_w + i, aw); else aw[0] = to_f32(a_w[i]);
#pragma unroll
                for (int e = 0; e < E; ++e) d[e] *= aw[e];
            }
#pragma unroll
            for (int e = 0; e < E; ++e) v[e] = fmaf(a_scale, d[e], v[e]);
        }
        if (br) {
#pragma unroll
            for (int e = 0; e < E; ++e) d[e] = 0.f;
            for (int s = 0; s < b_splits; ++s) {
                if constexpr (VEC) Quad<TD>::load(br + (size_t)s * b_stride + i, p); else p[0] = to_f32(br[(size_t)s * b_stride + i]);
#pragma unroll
                for (int e = 0; e < E; ++e) d[e] += p[e];
            }
#pragma unroll
            for (int e = 0; e < E; ++e) v[e] = fmaf(b_scale, d[e], v[e]);
        }
        if (write_back) {
            if constexpr (VEC) Quad<TX>::store(xr + i, v); else xr[i] = from_f32<TX>(v[0]);
        }
    };
    // the normed elements i .. i + E - 1
    const auto finish = [&](int i, const float (&v)[4], float mean, float inv) {
        float wv[4], o[4];
        if constexpr (VEC) Quad<TW>::load(w + i, wv); else wv[0] = to_f32(w[i]);
#pragma unroll
        for (int e = 0; e < E; ++e) o[e] = ((v[e] - mean) * inv) * wv[e];
        if (bias) {
            float bv[4];
            if constexpr (VEC) Quad<TW>::load(bias + i, bv); else bv[0] = to_f32(bias[i]);
#pragma unroll
            for (int e = 0; e < E; ++e) o[e] += bv[e];
        }
        if constexpr (VEC) Quad<TO>::store(orow + i, o); else orow[i] = from_f32<TO>(o[0]);
    };
    if constexpr (REG > 0) {
        float keep[REG][4];
#pragma unroll
        for (int q = 0; q < REG; ++q) gather((q * blockDim.x + threadIdx.x) * 4, keep[q]);
#pragma unroll
        for (int q = 0; q < REG; ++q)
#pragma unroll
            for (int e = 0; e < 4; ++e) sum += keep[q][e];
        const float mean = center ? block_sum(sum, scratch) / (float)len : 0.f;
        float ss = 0.f;
#pragma unroll
        for (int q = 0; q < REG; ++q)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float dd = keep[q][e] - mean;
                ss += dd * dd;
            }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)len + eps);
#pragma unroll
        for (int q = 0; q < REG; ++q) finish((q * blockDim.x + threadIdx.x) * 4, keep[q], mean, inv);
        return;
    }
    for (int i = threadIdx.x * E; i < len; i += blockDim.x * E) {
        float v[4];
        gather(i, v);
#pragma unroll
        for (int e = 0; e < E; ++e) {
            row_buf[i + e] = v[e];
            sum += v[e];
        }
    }
    const float mean = center ? block_sum(sum, scratch) / (float)len : 0.f;
    float ss = 0.f;
    for (int i = threadIdx.x * E; i < len; i += blockDim.x * E) {
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float dd = row_buf[i + e] - mean;
            ss += dd * dd;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)len + eps);
    for (int i = threadIdx.x * E; i < len; i += blockDim.x * E) {
        float v[4];
#pragma unroll
        for (int e = 0; e < E; ++e) v[e] = row_buf[i + e];
        finish(i, v, mean, inv);
    }
}

// x: [*, len] of x_dtype; a, b: null or stacks of delta_dtype; rows: null or n row indices (gather); w: [len] of w_dtype;
// out: [n, len] of out_dtype.  write_back stores the sum into x and needs rows == null.  bias, a_w: null or [len] of w_dtype.
static int run_layernorm(void* x, int x_dtype, const void* a, int a_splits, long long a_stride, float a_scale, const void* b, int b_splits,
                         long long b_stride, float b_scale, int delta_dtype, const int* rows, const void* w, int w_dtype, void* out, int out_dtype,
                         int n, int len, float eps, int write_back, int center, const void* bias, const void* a_w, const float* a_bias, const void* a_rows,
                         const float* a_row_w, cudaStream_t stream)
{
    if (n <= 0) return 0;
    if (len <= 0) SPY_FAIL("layernorm: row length %d must be positive", len);
    if (write_back && rows) SPY_FAIL("layernorm: write_back with a row gather is not defined");
    if ((a && a_splits <= 0) || (b && b_splits <= 0)) SPY_FAIL("layernorm: a stack of partial sums needs a positive number of parts");
    if (write_back && !a && !b) write_back = 0;
    if (!a && !b) delta_dtype = x_dtype;
    const size_t smem = (size_t)(len + 33) * sizeof(float);
    if (smem > 227 * 1024) SPY_FAIL("layernorm: a row of %d elements does not fit in shared memory (limit %d)", len, (227 * 1024) / 4 - 33);
    const bool vec = len % 4 == 0 && a_stride % 4 == 0 && b_stride % 4 == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(w) |
                       reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(a_w) | reinterpret_cast<uintptr_t>(a_bias) | reinterpret_cast<uintptr_t>(a_rows)) & 15) == 0;
    // many rows: fewer threads a row (two quads each) and so more rows an SM at a time; few rows: the row spread as wide as it goes
    int threads = (len / (vec ? (n >= 512 ? 8 : 4) : 4) + 31) / 32 * 32;
    threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
    SPY_DISPATCH_DTYPE(x_dtype, TX, {
        SPY_DISPATCH_DTYPE(delta_dtype, TD, {
            SPY_DISPATCH_DTYPE(w_dtype, TW, {
                SPY_DISPATCH_DTYPE(out_dtype, TO, {
                    // rows of exactly one, two or four quads a thread stay in registers
                    const int reg = !vec ? 0 : (len == 4 * threads ? 1 : (len == 8 * threads ? 2 : (len == 16 * threads ? 4 : 0)));
                    auto kernel = reg == 1 ? layernorm_kernel<TX, TD, TW, TO, true, 1> : reg == 2 ? layernorm_kernel<TX, TD, TW, TO, true, 2>
                                : reg == 4 ? layernorm_kernel<TX, TD, TW, TO, true, 4>
                                : (vec ? layernorm_kernel<TX, TD, TW, TO, true, 0> : layernorm_kernel<TX, TD, TW, TO, false, 0>);
                    if (smem > 48 * 1024) SPY_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                    spy_launch(kernel, dim3(n), dim3(threads), smem, stream, (TX*)x, (const TD*)a, a_splits, a_stride, a_scale, (const TD*)b, b_splits,
                               b_stride, b_scale, rows, (const TW*)w, (TO*)out, len, eps, write_back, center, (const TW*)bias, (const TW*)a_w, a_bias, (const TO*)a_rows, a_row_w);
                })
            })
        })
    })
    SPY_CHECK_LAUNCH("layernorm");
    return 0;
}

extern "C" int spy_layernorm(void* x, int x_dtype, const void* a, int a_splits, long long a_stride, float a_scale, const void* b, int b_splits,
                             long long b_stride, float b_scale, int delta_dtype, const int* rows, const void* w, int w_dtype, void* out, int out_dtype,
                             int n, int len, float eps, int write_back, int center, cudaStream_t stream)
{
    return run_layernorm(x, x_dtype, a, a_splits, a_stride, a_scale, b, b_splits, b_stride, b_scale, delta_dtype, rows, w, w_dtype, out, out_dtype, n, len,
                         eps, write_back, center, nullptr, nullptr, nullptr, nullptr, nullptr, stream);
}

// The same with a bias behind the weight and a per-channel multiplier of the first result (each null or [len] of w_dtype), and a
// bias of the first result itself (null or [len] float32).
extern "C" int spy_layernorm_affine(void* x, int x_dtype, const void* a, int a_splits, long long a_stride, float a_scale, const void* a_w, const float* a_bias,
                                    const void* a_rows, const float* a_row_w, const void* b,
                                    int b_splits, long long b_stride, float b_scale, int delta_dtype, const int* rows, const void* w, const void* bias,
                                    int w_dtype, void* out, int out_dtype, int n, int len, float eps, int write_back, int center, cudaStream_t stream)
{
    if ((a_w != nullptr || a_bias != nullptr || a_rows != nullptr) && a == nullptr) SPY_FAIL("layernorm: a per-channel multiplier, a bias or a row term without a result to go with");
    if ((a_rows != nullptr) != (a_row_w != nullptr)) SPY_FAIL("layernorm: a row term comes with its weights");
    return run_layernorm(x, x_dtype, a, a_splits, a_stride, a_scale, b, b_splits, b_stride, b_scale, delta_dtype, rows, w, w_dtype, out, out_dtype, n, len,
                         eps, write_back, center, bias, a_w, a_bias, a_rows, a_row_w, stream);
}

// out = scale_a * sum_s a[s] + scale_b * sum_s b[s], element by element in 32-bit: the weighted sum of two results (each
// one array or a stack of partial sums) for a consumer that cannot form it itself.
template <typename TD>
__global__ void scaled_sum_kernel(float* __restrict__ out, const TD* __restrict__ a, int a_splits, long long a_stride, float a_scale,
                                  const TD* __restrict__ b, int b_splits, long long b_stride, float b_scale, long long total)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        float x = 0.f, y = 0.f;
        for (int s = 0; s < a_splits; ++s) x += to_f32(a[(size_t)s * a_stride + i]);
        for (int s = 0; s < b_splits; ++s) y += to_f32(b[(size_t)s * b_stride + i]);
        out[i] = fmaf(b_scale, y, a_scale * x);
    }
}

extern "C" int spy_scaled_sum(float* out, const void* a, int a_splits, long long a_stride, float a_scale, const void* b, int b_splits, long long b_stride,
                              float b_scale, int delta_dtype, long long total, cudaStream_t stream)
{
    if (total <= 0) return 0;
    if (!a || !b || a_splits <= 0 || b_splits <= 0) SPY_FAIL("scaled_sum: two results are needed");
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    SPY_DISPATCH_DTYPE(delta_dtype, TD, {
        spy_launch(scaled_sum_kernel<TD>, dim3((int)blocks), dim3(256), 0, stream, out, (const TD*)a, a_splits, a_stride, a_scale, (const TD*)b, b_splits,
                   b_stride, b_scale, total);
    })
    SPY_CHECK_LAUNCH("scaled_sum");
    return 0;
}
