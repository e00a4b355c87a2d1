// Token embedding: out[t, :] = table[ids[t], :], widened to the 32-bit residual stream.
// Replaces the reference's __cuda_embedding_kernel (spymaster2h/spyinfer
// src/backends/cuda/native/common.cuh:45-55): same gather, no scaling.
#include "common.cuh"

SPY_MODULE(spy_embedding)

template <typename TW>
__global__ void embedding_kernel(const TW* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                 int hidden, int vocab, int* status)
{
    pdl_enter();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) report_status(status, SPY_STATUS_BAD_TOKEN, t);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(src[i]);
}

extern "C" int spy_embedding(const void* table, int table_dtype, const int* ids, float* out, int tokens, int hidden, int vocab,
                             int* status, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) SPY_FAIL("embedding: hidden %d and vocab %d must be positive", hidden, vocab);
    SPY_DISPATCH_DTYPE(table_dtype, TW, {
        spy_launch(embedding_kernel<TW>, dim3(tokens), dim3(256), 0, stream, (const TW*)table, ids, out, hidden, vocab, status);
    })
    SPY_CHECK_LAUNCH("embedding");
    return 0;
}

// The same gather with a scale, plus a row of a second table that is chosen by the pair (previous token, token):
//   out[t, :] = table[ids[t], :] * scale + pairs[row, :],
//   row = (previous * mul_prev + ids[t] * mul_cur) mod buckets, or `buckets` (the table's last row) for a sequence's first token.
// The previous token of a portion's first token is the sequence's state: prev_state[state_slot[seq]], which the block of
// that first token reads and then overwrites with the portion's last token (one thread does both, so the order holds).
template <typename TW, typename TP>
__global__ void embedding_pairs_kernel(const TW* __restrict__ table, const TP* __restrict__ pairs, const int* __restrict__ ids, float* __restrict__ out,
                                       int hidden, int vocab, float scale, long long buckets, long long mul_prev, long long mul_cur,
                                       const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                                       const int* __restrict__ state_slot, int* prev_state, int num_slots, int* status)
{
    __shared__ long long row_s;
    pdl_enter();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    const bool bad = id < 0 || id >= vocab;
    if (threadIdx.x == 0) {
        const int seq = seq_of_token[t], first = q_start[seq];
        long long row = buckets;
        int prev = -1;
        if (t > first) prev = ids[t - 1];
        else {
            const int slot = state_slot[seq];
            if (slot >= 0 && slot < num_slots) {
                prev = prev_state[slot];
                prev_state[slot] = ids[q_start[seq + 1] - 1];
            }
        }
        if (positions[t] > 0 && prev >= 0 && prev < vocab && !bad) row = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
        row_s = row;
        if (bad) report_status(status, SPY_STATUS_BAD_TOKEN, t);
    }
    __syncthreads();
    if (bad) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * hidden;
    const TP* add = pairs + (size_t)row_s * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(src[i]) * scale + to_f32(add[i]);
}

template <typename TW>
__global__ void embedding_scaled_kernel(const TW* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out, int hidden, int vocab,
                                        float scale, int* status)
{
    pdl_enter();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) report_status(status, SPY_STATUS_BAD_TOKEN, t);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(src[i]) * scale;
}

// pairs == null: only the scale.  pairs: [buckets + 1, hidden] of pairs_dtype; prev_state: [num_slots] int32.
extern "C" int spy_embedding_scaled(const void* table, int table_dtype, const int* ids, float* out, int tokens, int hidden, int vocab, float scale,
                                    const void* pairs, int pairs_dtype, long long buckets, long long mul_prev, long long mul_cur, const int* positions,
                                    const int* seq_of_token, const int* q_start, const int* state_slot, int* prev_state, int num_slots, int* status,
                                    cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) SPY_FAIL("embedding: hidden %d and vocab %d must be positive", hidden, vocab);
    if (pairs == nullptr) {
        SPY_DISPATCH_DTYPE(table_dtype, TW, {
            spy_launch(embedding_scaled_kernel<TW>, dim3(tokens), dim3(256), 0, stream, (const TW*)table, ids, out, hidden, vocab, scale, status);
        })
        SPY_CHECK_LAUNCH("embedding (scaled)");
        return 0;
    }
    if (buckets <= 0 || mul_prev < 0 || mul_cur < 0) SPY_FAIL("embedding: the pair table needs a positive number of buckets and multipliers that are not negative");
    if (!positions || !seq_of_token || !q_start || !state_slot || !prev_state || num_slots <= 0)
        SPY_FAIL("embedding: the pair table needs the batch's positions, sequences, starts, slots and the previous-token state");
    SPY_DISPATCH_DTYPE(table_dtype, TW, {
        SPY_DISPATCH_DTYPE(pairs_dtype, TP, {
            spy_launch(embedding_pairs_kernel<TW, TP>, dim3(tokens), dim3(256), 0, stream, (const TW*)table, (const TP*)pairs, ids, out, hidden, vocab,
                       scale, buckets, mul_prev, mul_cur, positions, seq_of_token, q_start, state_slot, prev_state, num_slots, status);
        })
    })
    SPY_CHECK_LAUNCH("embedding (pairs)");
    return 0;
}

// stream[t, :] += table[ids[t], :] + row[:]  (either term optional), in 32-bit: a model that adds its embedding output, or a
// learned offset, to the residual stream again at a later point of its depth.
template <typename TW, typename TR>
__global__ void stream_add_kernel(float* __restrict__ stream, const TW* __restrict__ table, const int* __restrict__ ids, const TR* __restrict__ row,
                                  int hidden, int vocab, int* status)
{
    pdl_enter();
    const int t = blockIdx.x;
    float* dst = stream + (size_t)t * hidden;
    const TW* src = nullptr;
    if (table != nullptr) {
        const int id = ids[t];
        if (id < 0 || id >= vocab) {
            if (threadIdx.x == 0) report_status(status, SPY_STATUS_BAD_TOKEN, t);
        } else {
            src = table + (size_t)id * hidden;
        }
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = dst[i];
        if (src != nullptr) v += to_f32(src[i]);
        if (row != nullptr) v += to_f32(row[i]);
        dst[i] = v;
    }
}

extern "C" int spy_stream_add(float* stream, const void* table, int table_dtype, const int* ids, const void* row, int row_dtype, int tokens, int hidden,
                              int vocab, int* status, cudaStream_t stream_)
{
    if (tokens <= 0 || (table == nullptr && row == nullptr)) return 0;
    if (hidden <= 0) SPY_FAIL("stream_add: hidden %d must be positive", hidden);
    if (table == nullptr) table_dtype = SPY_F32;
    if (row == nullptr) row_dtype = SPY_F32;
    SPY_DISPATCH_DTYPE(table_dtype, TW, {
        SPY_DISPATCH_DTYPE(row_dtype, TR, {
            spy_launch(stream_add_kernel<TW, TR>, dim3(tokens), dim3(256), 0, stream_, stream, (const TW*)table, ids, (const TR*)row, hidden, vocab, status);
        })
    })
    SPY_CHECK_LAUNCH("stream_add");
    return 0;
}
