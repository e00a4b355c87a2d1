// RMS norm in groups, with the residual sum of a normed sublayer output fused in.
//
// A row of `len` elements is cut into `groups` equal consecutive parts; each part is divided by its own
// sqrt(mean(part^2) + eps) and the whole row is multiplied by a weight.  One launch does, per row, either or both of
//   1. hidden += y_scale * group_norm(y) * y_weight      (y: a sublayer's output, possibly a stack of split-K partial sums)
//   2. out = group_norm(hidden) * weight                  (what the next sublayer reads, or the rows the head reads)
// with every statistic, the sum and the stream itself in 32-bit.  With `rows` the listed rows are gathered, normed into
// out[0..n) and nothing is written back.  One block a row; the row lives in shared memory between the steps.  The sums of
// squares are added in an order that depends only on the block size.
#include "common.cuh"

SPY_MODULE(spy_group_norm)

constexpr int GN_MAX_GROUPS = 64;
constexpr int GN_MAX_WARPS = 8;

// sum of squares of every group of row[0..len): result in sums[0..groups), visible to all threads on return
__device__ __forceinline__ void group_square_sums(const float* row, int len, int groups, float* part, float* sums)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5, gsz = len / groups;
    for (int g = 0; g < groups; ++g) {
        float s = 0.f;
        const float* r = row + g * gsz;
        for (int i = threadIdx.x; i < gsz; i += blockDim.x) s = fmaf(r[i], r[i], s);
        s = warp_sum(s);
        if (lane == 0) part[g * GN_MAX_WARPS + warp] = s;
    }
    __syncthreads();
    for (int g = threadIdx.x; g < groups; g += blockDim.x) {
        float s = 0.f;
        for (int w = 0; w < nwarps; ++w) s += part[g * GN_MAX_WARPS + w];
        sums[g] = s;
    }
    __syncthreads();
}

template <typename TY, typename TW, typename TO>
__global__ void group_norm_kernel(float* __restrict__ hidden, const TY* __restrict__ y, int splits, long long split_stride,
                                  const TW* __restrict__ y_weight, float y_scale, const int* __restrict__ rows,
                                  const TW* __restrict__ weight, TO* __restrict__ out, int len, int groups, float eps, int write_back)
{
    extern __shared__ float sm[];
    float* row = sm;                                    // len
    float* part = sm + len;                             // groups * GN_MAX_WARPS
    float* sums = part + groups * GN_MAX_WARPS;         // groups
    pdl_enter();
    const int r = blockIdx.x;
    const long long src = rows != nullptr ? rows[r] : r;
    const int gsz = len / groups;
    const float inv = 1.0f / (float)gsz;
    float* h = hidden + src * len;
    if (y != nullptr) {
        for (int i = threadIdx.x; i < len; i += blockDim.x) {
            float v = 0.f;
            for (int s = 0; s < splits; ++s) v += to_f32(y[s * split_stride + src * len + i]);
            row[i] = v;
        }
        __syncthreads();
        group_square_sums(row, len, groups, part, sums);
        for (int i = threadIdx.x; i < len; i += blockDim.x) {
            const float rstd = 1.0f / sqrtf(sums[i / gsz] * inv + eps);
            const float x = h[i] + y_scale * (row[i] * rstd * to_f32(y_weight[i]));
            row[i] = x;
            if (write_back) h[i] = x;
        }
    } else {
        for (int i = threadIdx.x; i < len; i += blockDim.x) row[i] = h[i];
    }
    if (weight == nullptr) return;
    __syncthreads();
    group_square_sums(row, len, groups, part, sums);
    TO* o = out + (long long)r * len;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        const float rstd = 1.0f / sqrtf(sums[i / gsz] * inv + eps);
        o[i] = from_f32<TO>(row[i] * rstd * to_f32(weight[i]));
    }
}

template <typename TY, typename TW, typename TO>
static int launch_group_norm(float* hidden, const void* y, int splits, long long split_stride, const void* y_weight, float y_scale, const int* rows,
                             const void* weight, void* out, int n, int len, int groups, float eps, int write_back, cudaStream_t stream)
{
    const size_t smem = ((size_t)len + (size_t)groups * (GN_MAX_WARPS + 1)) * sizeof(float);
    if (smem > 200 * 1024) SPY_FAIL("group_norm: a row of %d elements does not fit a block's shared memory", len);
    static size_t allowed[SPY_MAX_DEVICES] = {};
    const int dev = spy_device();
    if (smem > 48 * 1024 && allowed[dev] < smem) {
        SPY_CUDA(cudaFuncSetAttribute(group_norm_kernel<TY, TW, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        allowed[dev] = smem;
    }
    const int threads = len >= 2048 ? 256 : 128;
    spy_launch(group_norm_kernel<TY, TW, TO>, dim3(n), dim3(threads), smem, stream, hidden, (const TY*)y, splits, split_stride, (const TW*)y_weight,
               y_scale, rows, (const TW*)weight, (TO*)out, len, groups, eps, write_back);
    SPY_CHECK_LAUNCH("group_norm");
    return 0;
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
