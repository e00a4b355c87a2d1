// Causal convolution over time on each channel, with the inputs before a step's first token kept as per-request state.
//
//   conv(x)_t[c] = sum_j kernel[c, j] * x_(t - taps + 1 + j)[c]      (the kernel's last column meets the current token;
//                                                                     zeros stand before the sequence's start)
//   out_t[c] = act(conv(x)_t[c] + bias[c] (+ x_t[c] when `residual`))
//
// A step brings, for each request, a run of consecutive tokens that continues where the last step ended: the `taps - 1`
// inputs before the run are read from state[slot] (float32 [taps - 1, channels], oldest first, zero for a new request)
// and the run's last `taps - 1` inputs (or, for a shorter run, what is left of the old ones and the run) are stored there.
// Grid: y = channel tiles, x = request x piece of `piece` tokens; a thread owns one channel of one piece and walks its
// tokens with the last inputs in registers.  Only the thread of a run's first piece reads and writes the state of its
// (request, channel), so no thread reads what another writes.  Everything is computed in 32-bit.
#include "common.cuh"

SPY_MODULE(spy_time_conv)

constexpr int TC_PIECE = 16;       // tokens a thread walks; at least taps - 1, so that only a run's first piece needs the state

template <int MAXT, typename TI, typename TK, typename TO>
__global__ void time_conv_kernel(const TI* __restrict__ in, long long ld_in, const TK* __restrict__ kernel, const TK* __restrict__ bias,
                                 float* __restrict__ state, const int* __restrict__ q_start, const int* __restrict__ state_slot, TO* __restrict__ out,
                                 long long ld_out, int channels, int taps, int pieces, int residual, int act)
{
    pdl_enter();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int seq = blockIdx.x / pieces, piece = blockIdx.x % pieces;
    const int start = q_start[seq], end = q_start[seq + 1];
    const int t0 = start + piece * TC_PIECE, t1 = min(end, t0 + TC_PIECE);
    if (c >= channels || t0 >= end) return;
    const int hist_n = taps - 1;
    float k[MAXT], hist[MAXT];          // hist[i]: the input (taps - 1 - i) tokens back; hist[taps - 1] is unused
#pragma unroll
    for (int j = 0; j < MAXT; ++j) {
        k[j] = j < taps ? to_f32(kernel[(long long)c * taps + j]) : 0.f;
        hist[j] = 0.f;
    }
    const float b = bias != nullptr ? to_f32(bias[c]) : 0.f;
    if (piece == 0) {
        float* st = state + (long long)state_slot[seq] * hist_n * channels;
#pragma unroll
        for (int i = 0; i < MAXT - 1; ++i)
            if (i < hist_n) hist[i] = st[(long long)i * channels + c];
        // what the next step will find: the inputs at the run's last taps - 1 places, older ones taken from the old state
        const int n = end - start;
#pragma unroll
        for (int i = 0; i < MAXT - 1; ++i) {
            if (i < hist_n) {
                const int t = end - hist_n + i;
                float v;
                if (t >= start) v = to_f32(in[(long long)t * ld_in + c]);
                else {
                    v = 0.f;
#pragma unroll
                    for (int o = 0; o < MAXT - 1; ++o)
                        if (o == i + n) v = hist[o];
                }
                st[(long long)i * channels + c] = v;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < MAXT - 1; ++i)
            if (i < hist_n) hist[i] = to_f32(in[(long long)(t0 - hist_n + i) * ld_in + c]);
    }
    // four tokens' inputs are requested together, then used in order
    for (int tb = t0; tb < t1; tb += 4) {
        float xs[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) xs[u] = tb + u < t1 ? to_f32(in[(long long)(tb + u) * ld_in + c]) : 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int t = tb + u;
            if (t >= t1) break;
            const float x = xs[u];
            float acc = b;
#pragma unroll
            for (int i = 0; i < MAXT - 1; ++i)
                if (i < hist_n) acc = fmaf(k[i], hist[i], acc);
#pragma unroll
            for (int j = 0; j < MAXT; ++j)
                if (j == hist_n) acc = fmaf(k[j], x, acc);
            if (residual) acc += x;
            if (act == 1) acc = acc / (1.0f + expf(-acc));
            out[(long long)t * ld_out + c] = from_f32<TO>(acc);
#pragma unroll
            for (int i = 0; i < MAXT - 1; ++i) {
                if (i + 1 < hist_n) hist[i] = hist[i + 1];
                else if (i + 1 == hist_n) hist[i] = x;
            }
        }
    }
}

// in [T, ld_in] (its first `channels` columns are read), kernel [channels, taps], bias [channels] or none, state
// [slots, taps - 1, channels] float32, out [T, ld_out].  `longest`: no request brings more tokens than this.
// act: 0 none, 1 silu.
extern "C" int spy_time_conv(const void* in, int in_dtype, long long ld_in, const void* kernel, const void* bias, int kernel_dtype, float* state,
                             const int* q_start, const int* state_slot, int seqs, int longest, void* out, int out_dtype, long long ld_out,
                             int channels, int taps, int residual, int act, cudaStream_t stream)
{
    if (seqs <= 0 || longest <= 0) return 0;
    if (channels <= 0 || taps < 1 || taps > 16) SPY_FAIL("time_conv: %d channels and %d taps (1 to 16) are not served", channels, taps);
    if (taps > 1 && state == nullptr) SPY_FAIL("time_conv: %d taps need a state", taps);
    if (act < 0 || act > 1) SPY_FAIL("time_conv: unknown activation code %d", act);
    const int pieces = (longest + TC_PIECE - 1) / TC_PIECE;
    const long long rows = (long long)seqs * pieces;
    if (rows > 0x7fffffffLL || (channels + 127) / 128 > 65535) SPY_FAIL("time_conv: %d requests of up to %d tokens, %d channels exceed the grid", seqs, longest, channels);
    const dim3 grid((unsigned)rows, (channels + 127) / 128), block(128);
    SPY_DISPATCH_DTYPE(in_dtype, TI, {
        SPY_DISPATCH_DTYPE(kernel_dtype, TK, {
            SPY_DISPATCH_DTYPE(out_dtype, TO, {
                if (taps <= 4)
                    spy_launch(time_conv_kernel<4, TI, TK, TO>, grid, block, 0, stream, (const TI*)in, ld_in, (const TK*)kernel, (const TK*)bias, state,
                               q_start, state_slot, (TO*)out, ld_out, channels, taps, pieces, residual, act);
                else
                    spy_launch(time_conv_kernel<16, TI, TK, TO>, grid, block, 0, stream, (const TI*)in, ld_in, (const TK*)kernel, (const TK*)bias, state,
                               q_start, state_slot, (TO*)out, ld_out, channels, taps, pieces, residual, act);
            })
        })
    })
    SPY_CHECK_LAUNCH("time_conv");
    return 0;
}
