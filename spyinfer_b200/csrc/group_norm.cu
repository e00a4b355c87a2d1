// RMS norm in groups, with the residual sum of a normed sublayer output fused in.
//
// A row of `len` elements is cut into `groups` equal consecutive parts; each part is divided by its own
// sqrt(mean(part^2) + eps) and the whole row is multiplied by a weight.  One launch does, per row, either or both of
//   1. hidden += y_scale * group_norm(y) * y_weight      (y: a sublayer's output, possibly a stack of split-K partial sums)
//   2. out = group_norm(hidden) * weight                  (what the next sublayer reads, or the rows the head reads)
// with every statistic, the sum and the stream itself in 32-bit.  With `rows` the listed rows are gathered, normed into
// out[0..n) and nothing is written back.  One block a row; the row lives in shared memory between the steps.  The sums of
// squares are added in an order that depends only on the row's and the groups' lengths.
#include "common.cuh"

SPY_MODULE(spy_group_norm)

constexpr int GN_MAX_GROUPS = 64;
constexpr int GN_MAX_WARPS = 8;

// V consecutive elements at a time: 16- and 8-byte accesses for V = 4, plain ones for V = 1
template <typename T, int V> struct Run;
template <typename T> struct Run<T, 1> {
    static __device__ __forceinline__ void load(const T* p, float (&v)[1]) { v[0] = to_f32(p[0]); }
    static __device__ __forceinline__ void store(T* p, const float (&v)[1]) { p[0] = from_f32<T>(v[0]); }
};
template <> struct Run<float, 4> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4])
    {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Run<bf16, 4> {
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

// the warps' sums of squares of every group (part[g][warp]) -> sums[0..groups), visible to all threads on return
__device__ __forceinline__ void finish_square_sums(int groups, const float* part, float* sums)
{
    const int nwarps = blockDim.x >> 5;
    __syncthreads();
    for (int g = threadIdx.x; g < groups; g += blockDim.x) {
        float s = 0.f;
        for (int w = 0; w < nwarps; ++w) s += part[g * GN_MAX_WARPS + w];
        sums[g] = s;
    }
    __syncthreads();
}

// Every pass over the row goes group by group, V elements a thread and step (a run of V elements lies within one group), and
// adds the squares of what it has just made, so the row is read from memory once and walked three times at most.
template <typename TY, typename TW, typename TO, int V>
__global__ void group_norm_kernel(float* __restrict__ hidden, const TY* __restrict__ y, int splits, long long split_stride,
                                  const TW* __restrict__ y_weight, float y_scale, const int* __restrict__ rows,
                                  const TW* __restrict__ weight, TO* __restrict__ out, int len, int groups, float eps, int write_back)
{
    extern __shared__ __align__(16) float sm[];
    float* row = sm;                                    // len
    float* part = sm + len;                             // groups * GN_MAX_WARPS
    float* sums = part + groups * GN_MAX_WARPS;         // groups
    pdl_enter();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x;
    const long long src = rows != nullptr ? rows[r] : r;
    const int gsz = len / groups;
    const float inv = 1.0f / (float)gsz;
    float* h = hidden + src * len;
    float v[V], a[V], w[V];
    if (y != nullptr) {
        for (int g = 0; g < groups; ++g) {
            float ss = 0.f;
            for (int i = g * gsz + threadIdx.x * V; i < (g + 1) * gsz; i += blockDim.x * V) {
                Run<TY, V>::load(y + src * len + i, v);
                for (int s = 1; s < splits; ++s) {
                    Run<TY, V>::load(y + s * split_stride + src * len + i, a);
#pragma unroll
                    for (int e = 0; e < V; ++e) v[e] += a[e];
                }
#pragma unroll
                for (int e = 0; e < V; ++e) ss = fmaf(v[e], v[e], ss);
                Run<float, V>::store(row + i, v);
            }
            ss = warp_sum(ss);
            if (lane == 0) part[g * GN_MAX_WARPS + warp] = ss;
        }
        finish_square_sums(groups, part, sums);
        for (int g = 0; g < groups; ++g) {
            const float rstd = y_scale / sqrtf(sums[g] * inv + eps);
            float ss = 0.f;
            for (int i = g * gsz + threadIdx.x * V; i < (g + 1) * gsz; i += blockDim.x * V) {
                Run<float, V>::load(row + i, v);
                Run<float, V>::load(h + i, a);
                Run<TW, V>::load(y_weight + i, w);
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    a[e] += v[e] * rstd * w[e];
                    ss = fmaf(a[e], a[e], ss);
                }
                Run<float, V>::store(row + i, a);
                if (write_back) Run<float, V>::store(h + i, a);
            }
            ss = warp_sum(ss);
            if (lane == 0) part[g * GN_MAX_WARPS + warp] = ss;
        }
    } else {
        for (int g = 0; g < groups; ++g) {
            float ss = 0.f;
            for (int i = g * gsz + threadIdx.x * V; i < (g + 1) * gsz; i += blockDim.x * V) {
                Run<float, V>::load(h + i, a);
#pragma unroll
                for (int e = 0; e < V; ++e) ss = fmaf(a[e], a[e], ss);
                Run<float, V>::store(row + i, a);
            }
            ss = warp_sum(ss);
            if (lane == 0) part[g * GN_MAX_WARPS + warp] = ss;
        }
    }
    if (weight == nullptr) return;
    finish_square_sums(groups, part, sums);
    TO* o = out + (long long)r * len;
    for (int g = 0; g < groups; ++g) {
        const float rstd = 1.0f / sqrtf(sums[g] * inv + eps);
        for (int i = g * gsz + threadIdx.x * V; i < (g + 1) * gsz; i += blockDim.x * V) {
            Run<float, V>::load(row + i, a);
            Run<TW, V>::load(weight + i, w);
#pragma unroll
            for (int e = 0; e < V; ++e) a[e] = a[e] * rstd * w[e];
            Run<TO, V>::store(o + i, a);
        }
    }
}

template <typename TY, typename TW, typename TO, int V>
static int launch_group_norm_v(float* hidden, const void* y, int splits, long long split_stride, const void* y_weight, float y_scale, const int* rows,
                               const void* weight, void* out, int n, int len, int groups, float eps, int write_back, cudaStream_t stream)
{
    const size_t smem = ((size_t)len + (size_t)groups * (GN_MAX_WARPS + 1)) * sizeof(float);
    if (smem > 200 * 1024) SPY_FAIL("group_norm: a row of %d elements does not fit a block's shared memory", len);
    static size_t allowed[SPY_MAX_DEVICES] = {};
    const int dev = spy_device();
    if (smem > 48 * 1024 && allowed[dev] < smem) {
        SPY_CUDA(cudaFuncSetAttribute(group_norm_kernel<TY, TW, TO, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        allowed[dev] = smem;
    }
    const int per_group = len / groups / V;                    // steps of one thread's work in a group
    const int threads = per_group >= 256 ? 256 : per_group >= 128 ? 128 : per_group >= 64 ? 64 : 32;
    spy_launch(group_norm_kernel<TY, TW, TO, V>, dim3(n), dim3(threads), smem, stream, hidden, (const TY*)y, splits, split_stride, (const TW*)y_weight,
               y_scale, rows, (const TW*)weight, (TO*)out, len, groups, eps, write_back);
    SPY_CHECK_LAUNCH("group_norm");
    return 0;
}

// Runs of four where every group is a multiple of four long (rows and groups then start on 16-byte borders of the 32-bit
// tensors and 8-byte borders of the bfloat16 ones) and the parts of a stack are as far apart.
template <typename TY, typename TW, typename TO>
static int launch_group_norm(float* hidden, const void* y, int splits, long long split_stride, const void* y_weight, float y_scale, const int* rows,
                             const void* weight, void* out, int n, int len, int groups, float eps, int write_back, cudaStream_t stream)
{
    auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = (len / groups) % 4 == 0 && split_stride % 4 == 0 && aligned(hidden) && aligned(y) && aligned(y_weight) && aligned(weight) && aligned(out);
    if (vec)
        return launch_group_norm_v<TY, TW, TO, 4>(hidden, y, splits, split_stride, y_weight, y_scale, rows, weight, out, n, len, groups, eps, write_back, stream);
    return launch_group_norm_v<TY, TW, TO, 1>(hidden, y, splits, split_stride, y_weight, y_scale, rows, weight, out, n, len, groups, eps, write_back, stream);
}

// hidden [*, len] float32.  y (optional): [splits][rows][len] of y_dtype with its weight and scale.  weight/out (optional):
// the norm of the (new) stream rows into out [n, len] of out_dtype.  Both weights have weight_dtype.
extern "C" int spy_group_norm(float* hidden, const void* y, int y_dtype, int splits, long long split_stride, const void* y_weight, float y_scale,
                              const int* rows, const void* weight, int weight_dtype, void* out, int out_dtype, int n, int len, int groups, float eps,
                              int write_back, cudaStream_t stream)
{
    if (n <= 0) return 0;
    if (len <= 0 || groups <= 0 || groups > GN_MAX_GROUPS || len % groups != 0)
        SPY_FAIL("group_norm: a row of %d elements cannot be cut into %d equal groups (at most %d)", len, groups, GN_MAX_GROUPS);
    if (y == nullptr && weight == nullptr) return 0;
    if (y != nullptr && (y_weight == nullptr || splits < 1)) SPY_FAIL("group_norm: a sublayer output needs its weight and at least one part");
    if (weight != nullptr && out == nullptr) SPY_FAIL("group_norm: a norm needs an output");
    if (y == nullptr) y_dtype = SPY_F32;
    if (out == nullptr) out_dtype = SPY_F32;
    SPY_DISPATCH_DTYPE(y_dtype, TY, {
        SPY_DISPATCH_DTYPE(weight_dtype, TW, {
            SPY_DISPATCH_DTYPE(out_dtype, TO, {
                return launch_group_norm<TY, TW, TO>(hidden, y, splits, split_stride, y_weight, y_scale, rows, weight, out, n, len, groups, eps,
                                                     write_back, stream);
            })
        })
    })
    return 0;
}
