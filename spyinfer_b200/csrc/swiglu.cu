// SwiGLU on a fused gate|up activation: out[t, i] = silu(x[t, i]) * x[t, inter + i],
// silu(g) = g / (1 + exp(-g)), computed in 32-bit.  Replaces the reference's
// __cuda_swiglu_fp16 (spymaster2h/spyinfer src/backends/cuda/native/common.cu:56-73), which
// works in half arithmetic on separate gate and up tensors.
#include "common.cuh"

SPY_MODULE(spy_swiglu)

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, long long total)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const long long row = i / inter;
        const int col = (int)(i - row * inter);
        const T* src = gate_up + row * 2 * inter;
        const float g = to_f32(src[col]);
        const float u = to_f32(src[inter + col]);
        out[i] = from_f32<T>((g / (1.0f + expf(-g))) * u);
    }
}

extern "C" int spy_swiglu(const void* gate_up, void* out, int dtype, int tokens, int inter, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (inter <= 0) SPY_FAIL("swiglu: intermediate size %d must be positive", inter);
    const long long total = (long long)tokens * inter;
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    SPY_DISPATCH_DTYPE(dtype, T, {
        spy_launch(swiglu_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (const T*)gate_up, (T*)out, inter, total);
    })
    SPY_CHECK_LAUNCH("swiglu");
    return 0;
}

// out[t, c] += bias[c], in 32-bit: the bias of a product whose kernel has no bias term of its own
// (the reference's linear adds one when it is bound, spymaster2h/spyinfer
// src/backends/cpu/cpu_operator.cpp:150-186; its model binds none, src/models/qwen3.hpp:39, 143).
template <typename T, typename TB>
__global__ void add_bias_kernel(T* __restrict__ out, const TB* __restrict__ bias, int cols, long long total)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) out[i] = from_f32<T>(to_f32(out[i]) + to_f32(bias[i % cols]));
}

extern "C" int spy_add_bias(void* out, int dtype, const void* bias, int bias_dtype, int rows, int cols, cudaStream_t stream)
{
    if (rows <= 0) return 0;
    if (cols <= 0) SPY_FAIL("add_bias: %d columns", cols);
    const long long total = (long long)rows * cols;
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    SPY_DISPATCH_DTYPE(dtype, T, {
        SPY_DISPATCH_DTYPE(bias_dtype, TB, {
            spy_launch(add_bias_kernel<T, TB>, dim3((int)blocks), dim3(256), 0, stream, (T*)out, (const TB*)bias, cols, total);
        })
    })
    SPY_CHECK_LAUNCH("add_bias");
    return 0;
}


// out[i] = act(x[i]) element by element in 32-bit: the activation of a feed-forward without a gate.
//   0: relu(x)^2    1: gelu with the tanh approximation, 0.5 x (1 + tanh(sqrt(2 / pi) (x + 0.044715 x^3)))    2: silu    3: relu
template <typename T>
__global__ void activation_kernel(const T* __restrict__ x, T* __restrict__ out, long long total, int act)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const float v = to_f32(x[i]);
        float r;
        if (act == 0) { const float p = fmaxf(v, 0.f); r = p * p; }
        else if (act == 1) r = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        else if (act == 2) r = v / (1.0f + expf(-v));
        else r = fmaxf(v, 0.f);
        out[i] = from_f32<T>(r);
    }
}

extern "C" int spy_activation(const void* x, void* out, int dtype, long long total, int act, cudaStream_t stream)
{
    if (total <= 0) return 0;
    if (act < 0 || act > 3) SPY_FAIL("activation: unknown code %d", act);
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    SPY_DISPATCH_DTYPE(dtype, T, {
        spy_launch(activation_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (const T*)x, (T*)out, total, act);
    })
    SPY_CHECK_LAUNCH("activation");
    return 0;
}

// x[i] *= scale in place (32-bit): a model whose logits carry a multiplier.
__global__ void scale_kernel(float* __restrict__ x, long long total, float scale)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) x[i] *= scale;
}

extern "C" int spy_scale(float* x, long long total, float scale, cudaStream_t stream)
{
    if (total <= 0) return 0;
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    spy_launch(scale_kernel, dim3((int)blocks), dim3(256), 0, stream, x, total, scale);
    SPY_CHECK_LAUNCH("scale");
    return 0;
}

// A gated activation on a fused gate|up tensor: out[t, i] = act(x[t, i]) * x[t, inter + i] in 32-bit.
//   0: silu    1: gelu with the tanh approximation
template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, long long total, int act)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const long long row = i / inter;
        const int col = (int)(i - row * inter);
        const T* src = gate_up + row * 2 * inter;
        const float g = to_f32(src[col]);
        const float u = to_f32(src[inter + col]);
        const float a = act == 0 ? g / (1.0f + expf(-g)) : 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
        out[i] = from_f32<T>(a * u);
    }
}

extern "C" int spy_gated_activation(const void* gate_up, void* out, int dtype, int tokens, int inter, int act, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (inter <= 0 || act < 0 || act > 1) SPY_FAIL("gated_activation: intermediate size %d, activation code %d", inter, act);
    const long long total = (long long)tokens * inter;
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    SPY_DISPATCH_DTYPE(dtype, T, {
        spy_launch(gated_activation_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (const T*)gate_up, (T*)out, inter, total, act);
    })
    SPY_CHECK_LAUNCH("gated_activation");
    return 0;
}

// A clamped gated activation on a fused gate|up tensor with the projections' bias folded in (32-bit arithmetic):
//   g = min(x[t, i] + b[i], limit), u = clamp(x[t, inter + i] + b[inter + i], -limit, limit), out[t, i] = g * sigmoid(alpha * g) * (u + 1).
// bias: null or [2 * inter] float32.  TI, TO: the input's and the output's type (a 32-bit product may feed a bfloat16 activation).
template <typename TI, typename TO>
__global__ void clamped_glu_kernel(const TI* __restrict__ gate_up, const float* __restrict__ bias, TO* __restrict__ out, int inter, long long total,
                                   float limit, float alpha)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const long long row = i / inter;
        const int col = (int)(i - row * inter);
        const TI* src = gate_up + row * 2 * inter;
        float g = to_f32(src[col]), u = to_f32(src[inter + col]);
        if (bias != nullptr) {
            g += bias[col];
            u += bias[inter + col];
        }
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        out[i] = from_f32<TO>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
    }
}

// The same, four neighbouring outputs a thread (inter, and with it every row pitch, a multiple of 4; arrays aligned for 4-element accesses).
template <typename TI, typename TO>
__global__ void clamped_glu_quads_kernel(const TI* __restrict__ gate_up, const float* __restrict__ bias, TO* __restrict__ out, int inter, long long quads,
                                         float limit, float alpha)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const int per_row = inter / 4;
    for (; i < quads; i += stride) {
        const long long row = i / per_row;
        const int col = (int)(i - row * per_row) * 4;
        const TI* src = gate_up + row * 2 * inter;
        float g[4], u[4], o[4];
        if constexpr (sizeof(TI) == 4) {
            const float4 a = *reinterpret_cast<const float4*>(src + col), b = *reinterpret_cast<const float4*>(src + inter + col);
            g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; u[0] = b.x; u[1] = b.y; u[2] = b.z; u[3] = b.w;
        } else {
            const uint2 a = *reinterpret_cast<const uint2*>(src + col), b = *reinterpret_cast<const uint2*>(src + inter + col);
            const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
            g[0] = __low2float(a2[0]); g[1] = __high2float(a2[0]); g[2] = __low2float(a2[1]); g[3] = __high2float(a2[1]);
            u[0] = __low2float(b2[0]); u[1] = __high2float(b2[0]); u[2] = __low2float(b2[1]); u[3] = __high2float(b2[1]);
        }
        if (bias != nullptr) {
            const float4 bg = *reinterpret_cast<const float4*>(bias + col), bu = *reinterpret_cast<const float4*>(bias + inter + col);
            g[0] += bg.x; g[1] += bg.y; g[2] += bg.z; g[3] += bg.w; u[0] += bu.x; u[1] += bu.y; u[2] += bu.z; u[3] += bu.w;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float gg = fminf(g[e], limit), uu = fminf(fmaxf(u[e], -limit), limit);
            o[e] = gg / (1.0f + expf(-alpha * gg)) * (uu + 1.0f);
        }
        if constexpr (sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(out + i * 4) = make_float4(o[0], o[1], o[2], o[3]);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
            uint2 x;
            x.x = *reinterpret_cast<uint32_t*>(&lo);
            x.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(out + i * 4) = x;
        }
    }
}

extern "C" int spy_clamped_glu(const void* gate_up, int in_dtype, const float* bias, void* out, int out_dtype, int tokens, int inter, float limit,
                               float alpha, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (inter <= 0 || !(limit > 0.f)) SPY_FAIL("clamped_glu: intermediate size %d, limit %g", inter, (double)limit);
    const long long total = (long long)tokens * inter;
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    const bool quads = inter % 4 == 0 && ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(bias)) & 15) == 0;
    if (quads) {
        blocks = (total / 4 + 255) / 256;
        if (blocks > most) blocks = most;
    }
    SPY_DISPATCH_DTYPE(in_dtype, TI, {
        SPY_DISPATCH_DTYPE(out_dtype, TO, {
            if (quads)
                spy_launch(clamped_glu_quads_kernel<TI, TO>, dim3((int)blocks), dim3(256), 0, stream, (const TI*)gate_up, bias, (TO*)out, inter, total / 4, limit,
                           alpha);
            else
                spy_launch(clamped_glu_kernel<TI, TO>, dim3((int)blocks), dim3(256), 0, stream, (const TI*)gate_up, bias, (TO*)out, inter, total, limit, alpha);
        })
    })
    SPY_CHECK_LAUNCH("clamped_glu");
    return 0;
}

// x[i] = cap * tanh(x[i] / cap) in place (32-bit): logits with a soft cap.
__global__ void softcap_kernel(float* __restrict__ x, long long total, float cap)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) x[i] = cap * tanhf(x[i] / cap);
}

extern "C" int spy_softcap(float* x, long long total, float cap, cudaStream_t stream)
{
    if (total <= 0) return 0;
    if (!(cap > 0.f)) SPY_FAIL("softcap: the cap %g must be positive", (double)cap);
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    spy_launch(softcap_kernel, dim3((int)blocks), dim3(256), 0, stream, x, total, cap);
    SPY_CHECK_LAUNCH("softcap");
    return 0;
}
