// The real-gated linear recurrent unit of a Griffin-style recurrent block, over packed steps of several sequences.
//
// The block's two input projections arrive as one float matrix yx [tokens, row_stride]: channels 0 .. C-1 are the
// gate branch before its bias and activation, channels x_offset .. x_offset + C-1 the recurrent branch before its
// bias.  Per channel c and position p of a sequence:
//
//   xb_p  = x_p + x_bias                                   u_p = conv_b + sum_k conv_w[c, k] * xb_(p - (taps-1-k))
//   r, i  = sigmoid(block-diagonal matrices on u + biases)  (the matrix products are headwise_linear's)
//   a     = exp(-8 * r * softplus(lam))                     S_p = a * S_(p-1) + sqrt(1 - a^2) * i * u_p
//   out_p = S_p * gelu_tanh(y_p + y_bias)                   (compute dtype: the input of the output projection)
//
// Everything here is float.  Per sequence the cache keeps float state, one row per slot:
//   [2][C]     S after the last position, in the half chosen by that position's parity: a step reads the half of
//              the position before its first and writes the half of its last, so a one-token step that runs twice
//              (a graph's capture after its warm-up) computes the same thing both times;
//   [taps][C]  xb of the last `taps` positions, at row (position mod taps): a one-token step writes the row that
//              none of its own taps reads.
// Positions before a sequence's start count as zero input and zero state.
#include "common.cuh"

namespace skv {

constexpr float RGLRU_DECAY_SCALE = 8.0f;

struct RecurrentBatch {
    const int* positions;      // [tokens]
    const int* token_seq;      // [tokens]
    const int* cu_q;           // [seqs + 1]
    const int* slot_ids;       // [seqs]
    float* state;              // [slots][state_stride]
    int state_stride;          // floats per slot: (2 + taps) * C
};

// u[t, c]: a block row per token (what is known per token is looked up once a block), threads over the channels.
__global__ void __launch_bounds__(256)
rglru_conv_kernel(const float* __restrict__ yx, int row_stride, int x_offset, const float* __restrict__ x_bias,
                  const float* __restrict__ conv_w, const float* __restrict__ conv_b, float* __restrict__ u,
                  int first_token, int channels, int taps, const RecurrentBatch batch) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = first_token + blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int p = batch.positions[t], s = batch.token_seq[t];
    const int first = batch.cu_q[s];
    const float* ring = batch.state + (size_t)batch.slot_ids[s] * batch.state_stride + 2 * (size_t)channels;
    const float bias = x_bias[c];
    float sum = conv_b[c];
    for (int k = 0; k < taps; ++k) {
        const int back = taps - 1 - k;
        if (p - back < 0) continue;
        const float v = t - back >= first ? yx[(size_t)(t - back) * row_stride + x_offset + c] + bias
                                          : ring[(size_t)((p - back) % taps) * channels + c];
        sum = fmaf(conv_w[(size_t)c * taps + k], v, sum);
    }
    u[(size_t)t * channels + c] = sum;
}

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// rate[c] = 8 * softplus(lam[c]): the part of the decay's exponent that does not depend on the token, made once when
// the weights are loaded.
__global__ void rglru_rate_kernel(const float* __restrict__ lam, float* __restrict__ rate, int channels) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < channels) rate[c] = RGLRU_DECAY_SCALE * softplus_f(lam[c]);
}

// Per (token, channel): from the gates' matrix products (gates [tokens, 2C]: per part of `part` channels first the
// part's r rows, then its i rows) to the decay a and the driven input sqrt(1 - a^2) * i * u, which replace them in
// place; and the gate branch's activation in place of its pre-activation in yx.
__global__ void __launch_bounds__(256)
rglru_gates_kernel(float* __restrict__ gates, const float* __restrict__ u, float* __restrict__ yx, int row_stride,
                   const float* __restrict__ y_bias, const float* __restrict__ r_bias,
                   const float* __restrict__ i_bias, const float* __restrict__ rate, int n_tokens, int channels,
                   int part) {
    pdl_launch_dependents();
    pdl_wait();
    const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= (long long)n_tokens * channels) return;
    const int t = (int)(item / channels), c = (int)(item - (long long)t * channels);
    const int b = c / part, within = c - b * part;
    float* pair = gates + (size_t)t * 2 * channels + (size_t)b * 2 * part + within;
    const float r = sigmoid_f(pair[0] + r_bias[c]);
    const float i = sigmoid_f(pair[part] + i_bias[c]);
    const float a = expf(-r * rate[c]);
    pair[0] = a;
    pair[part] = sqrtf(fmaxf(1.0f - a * a, 0.0f)) * i * u[(size_t)t * channels + c];
    float* y = yx + (size_t)t * row_stride + c;
    *y = gelu_tanh(*y + y_bias[c]);
}

// The recurrence.  A sequence's tokens of this step are cut into chunks of `chunk` tokens and a thread walks one
// chunk of one channel.  With more than one chunk a first pass (rglru_chunk_kernel) leaves for every chunk the product
// A of its decays and the state B that it reaches from zero; the chunk's true first state then follows from the state
// before the step and the (A, B) of the chunks in front: S <- A S + B, chunk by chunk.  So a prompt of thousands of
// tokens is tens of short walks side by side and not one long one.  `summary` is [seqs][max_chunks][2][C] floats.
__global__ void __launch_bounds__(128)
rglru_chunk_kernel(const float* __restrict__ gates, float* __restrict__ summary, int n_seqs, int channels, int part,
                   int chunk, int max_chunks, const int* __restrict__ cu_q) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y, k = blockIdx.z;
    if (c >= channels || s >= n_seqs) return;
    const int first = cu_q[s] + k * chunk, last = min(cu_q[s + 1] - 1, first + chunk - 1);
    if (first > last) return;
    const int b = c / part, within = c - b * part;
    const float* pair = gates + (size_t)b * 2 * part + within;
    float A = 1.0f, B = 0.0f;
#pragma unroll 4
    for (int t = first; t <= last; ++t) {
        const float a = pair[(size_t)t * 2 * channels], driven = pair[(size_t)t * 2 * channels + part];
        A *= a;
        B = fmaf(a, B, driven);
    }
    float* mine = summary + ((size_t)s * max_chunks + k) * 2 * channels;
    mine[c] = A;
    mine[channels + c] = B;
}

template <typename T>
__global__ void __launch_bounds__(128)
rglru_scan_kernel(const float* __restrict__ gates, const float* __restrict__ yx, int row_stride, int x_offset,
                  const float* __restrict__ x_bias, T* __restrict__ out, int out_stride, int n_seqs, int channels,
                  int part, int taps, int chunk, int max_chunks, const float* __restrict__ summary,
                  const RecurrentBatch batch) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y, k = blockIdx.z;
    if (c >= channels || s >= n_seqs) return;
    const int seq_first = batch.cu_q[s], seq_last = batch.cu_q[s + 1] - 1;
    const int first = seq_first + k * chunk, last = min(seq_last, first + chunk - 1);
    if (first > last) return;
    const int p_first = batch.positions[seq_first], p_last = p_first + (seq_last - seq_first);
    float* state = batch.state + (size_t)batch.slot_ids[s] * batch.state_stride;
    const int b = c / part, within = c - b * part;
    const float* pair = gates + (size_t)b * 2 * part + within;
    float S = p_first > 0 ? state[(size_t)((p_first - 1) & 1) * channels + c] : 0.0f;
    for (int j = 0; j < k; ++j) {                      // through the chunks in front of this one
        const float* theirs = summary + ((size_t)s * max_chunks + j) * 2 * channels;
        S = fmaf(theirs[c], S, theirs[channels + c]);
    }
#pragma unroll 4
    for (int t = first; t <= last; ++t) {
        const float a = pair[(size_t)t * 2 * channels], driven = pair[(size_t)t * 2 * channels + part];
        const float y = yx[(size_t)t * row_stride + c];
        S = fmaf(a, S, driven);
        out[(size_t)t * out_stride + c] = from_float<T>(S * y);
    }
    if (last != seq_last) return;                      // the sequence's last chunk leaves the state
    state[(size_t)(p_last & 1) * channels + c] = S;
    float* ring = state + 2 * (size_t)channels;
    const float bias = x_bias[c];
    for (int back = 0; back < taps && seq_last - back >= seq_first; ++back)
        ring[(size_t)((p_last - back) % taps) * channels + c] = yx[(size_t)(seq_last - back) * row_stride + x_offset + c] + bias;
}

}  // namespace skv

using namespace skv;

static int check_batch(const char* name, const int* positions, const int* token_seq, const int* cu_q,
                       const int* slot_ids, float* state, int state_stride, int channels, int taps) {
    if (!positions || !token_seq || !cu_q || !slot_ids || !state) return fail(name, "the step's metadata and the state are needed");
    if (channels <= 0 || taps <= 0) return fail(name, "channels and taps must be positive");
    if (state_stride < (2 + taps) * channels) return fail(name, "a slot's state is too small: (2 + taps) * channels floats are needed");
    return 0;
}

SKV_EXPORT int skv_rglru_conv(const float* yx, int row_stride, int x_offset, const float* x_bias, const float* conv_w,
                              const float* conv_b, float* u, int n_tokens, int channels, int taps,
                              const int* positions, const int* token_seq, const int* cu_q, const int* slot_ids,
                              float* state, int state_stride, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (int code = check_batch("skv_rglru_conv", positions, token_seq, cu_q, slot_ids, state, state_stride, channels, taps)) return code;
    if (x_offset < 0 || row_stride < x_offset + channels) return fail("skv_rglru_conv", "a row is shorter than its two branches");
    const RecurrentBatch batch = {positions, token_seq, cu_q, slot_ids, state, state_stride};
    // (grid.y holds 65,535 rows at most: longer steps go in pieces)
    for (int done = 0; done < n_tokens; done += 65535) {
        const int rows = n_tokens - done < 65535 ? n_tokens - done : 65535;
        if (int code = launch_pdl("skv_rglru_conv", rglru_conv_kernel, dim3((channels + 255) / 256, rows), dim3(256), 0, stream,
                                  yx, row_stride, x_offset, x_bias, conv_w, conv_b, u, done, channels, taps, batch))
            return code;
    }
    return 0;
}

// rate [channels] float = 8 * softplus(lam [channels] float).
SKV_EXPORT int skv_rglru_rate(const float* lam, float* rate, int channels, cudaStream_t stream) {
    if (channels <= 0) return 0;
    rglru_rate_kernel<<<(channels + 255) / 256, 256, 0, stream>>>(lam, rate, channels);
    return check_launch("skv_rglru_rate");
}

// `rate`: what skv_rglru_rate made of the layer's lam.
SKV_EXPORT int skv_rglru_gates(float* gates, const float* u, float* yx, int row_stride, const float* y_bias,
                               const float* r_bias, const float* i_bias, const float* rate, int n_tokens, int channels,
                               int part, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (channels <= 0 || part <= 0 || channels % part != 0) return fail("skv_rglru_gates", "the channels must split into equal parts");
    if (row_stride < channels) return fail("skv_rglru_gates", "a row is shorter than its channels");
    const long long blocks = ((long long)n_tokens * channels + 255) / 256;
    if (blocks > 0x7fffffffLL) return fail("skv_rglru_gates", "too many tokens in one step");
    return launch_pdl("skv_rglru_gates", rglru_gates_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, gates, u, yx,
                      row_stride, y_bias, r_bias, i_bias, rate, n_tokens, channels, part);
}

constexpr int RGLRU_CHUNK = 64;

// Floats of `summary` that a step whose longest sequence brings max_q_len tokens needs (0: none, it runs as one chunk).
SKV_EXPORT long long skv_rglru_scan_scratch(int n_seqs, int max_q_len, int channels) {
    if (max_q_len <= 2 * RGLRU_CHUNK) return 0;
    return (long long)n_seqs * ((max_q_len + RGLRU_CHUNK - 1) / RGLRU_CHUNK) * 2 * channels;
}

// out [tokens, out_stride] in the compute dtype: S * activated gate branch, the input of the output projection.
// max_q_len: the most tokens a sequence brings; summary: skv_rglru_scan_scratch floats (null where that is 0).
SKV_EXPORT int skv_rglru_scan(const float* gates, const float* yx, int row_stride, int x_offset, const float* x_bias,
                              void* out, int out_stride, int n_seqs, int channels, int part, int taps, int max_q_len,
                              float* summary,
                              const int* positions, const int* token_seq, const int* cu_q, const int* slot_ids,
                              float* state, int state_stride, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (int code = check_batch("skv_rglru_scan", positions, token_seq, cu_q, slot_ids, state, state_stride, channels, taps)) return code;
    if (part <= 0 || channels % part != 0) return fail("skv_rglru_scan", "the channels must split into equal parts");
    if (n_seqs > 65535) return fail("skv_rglru_scan", "too many sequences in one step");
    if (out_stride < channels) return fail("skv_rglru_scan", "a row of the output is shorter than its channels");
    const RecurrentBatch batch = {positions, token_seq, cu_q, slot_ids, state, state_stride};
    if (max_q_len <= 0) return fail("skv_rglru_scan", "the longest sequence's token count is needed");
    const bool chunked = skv_rglru_scan_scratch(n_seqs, max_q_len, channels) > 0;
    if (chunked && !summary) return fail("skv_rglru_scan", "a step this long needs scratch for its chunks");
    const int chunk = chunked ? RGLRU_CHUNK : max_q_len;
    const int max_chunks = (max_q_len + chunk - 1) / chunk;
    if (max_chunks > 65535) return fail("skv_rglru_scan", "too many tokens of one sequence in one step");
    const dim3 grid((channels + 127) / 128, n_seqs, max_chunks);
    if (chunked)
        if (int code = launch_pdl("skv_rglru_scan", rglru_chunk_kernel, grid, dim3(128), 0, stream, gates, summary, n_seqs,
                                  channels, part, chunk, max_chunks, cu_q))
            return code;
    return launch_pdl("skv_rglru_scan", rglru_scan_kernel<skv_t>, grid, dim3(128), 0,
                      stream, gates, yx, row_stride, x_offset, x_bias, (skv_t*)out, out_stride, n_seqs, channels, part,
                      taps, chunk, max_chunks, (const float*)summary, batch);
}
