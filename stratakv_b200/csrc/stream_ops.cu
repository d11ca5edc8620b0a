// Kernels on the float residual stream for layers that norm a sublayer's output before it is added, and for a
// per-layer input that depends on the token:
//
//   rmsnorm_add:  x[r, :] += y[r, :] / sqrt(mean(y[r, :]^2) + eps) * gamma          (the norm after a sublayer)
//   token_side:   e = table[token, offset : offset + dim];  g = gelu_tanh(gate_w . x) * e;  y = proj_w . g;
//                 x += y / sqrt(mean(y^2) + eps) * norm_w                            (dim is small: tens)
//
// Both can hand the next reader its input in the same pass: with next_out, the new row of the stream is normed
// with next_gamma and next_eps and written in the compute dtype, so the norm in front of the next sublayer needs no
// kernel of its own.  Everything is float but the tables and weights, which are read in the compute dtype.
#include "common.cuh"

namespace skv {

template <typename T>
__global__ void rmsnorm_add_kernel(const float* __restrict__ y, const float* __restrict__ gamma, float eps,
                                   float* __restrict__ x, const float* __restrict__ next_gamma, float next_eps,
                                   T* __restrict__ next_out, int hidden) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t r = blockIdx.x;
    const float* y_row = y + r * hidden;
    float* x_row = x + r * hidden;
    float partial = 0.0f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = y_row[c];
        partial = fmaf(v, v, partial);
    }
    const float inverse_rms = 1.0f / sqrtf(block_sum(partial, scratch) / (float)hidden + eps);
    float squares = 0.0f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = x_row[c] + y_row[c] * inverse_rms * gamma[c];
        x_row[c] = v;
        squares = fmaf(v, v, squares);
    }
    if (!next_out) return;
    const float next_inverse = 1.0f / sqrtf(block_sum(squares, scratch) / (float)hidden + next_eps);
    T* out_row = next_out + r * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)     // (each thread reads back what it wrote itself)
        out_row[c] = from_float<T>(x_row[c] * next_inverse * next_gamma[c]);
}

// A block takes SIDE_TOKENS tokens, so that it reads the two weights once for all of them: `proj_t` is the projection
// transposed, [dim][hidden], which lets neighbouring threads read neighbouring columns.
constexpr int SIDE_TOKENS = 4;

template <typename T>
__global__ void token_side_kernel(float* __restrict__ x, const int* __restrict__ ids, const T* __restrict__ table,
                                  int table_stride, int offset, int dim, int vocab, const T* __restrict__ gate_w,
                                  const T* __restrict__ proj_t, const float* __restrict__ norm_w, float eps,
                                  const float* __restrict__ next_gamma, float next_eps, T* __restrict__ next_out,
                                  int n_tokens, int hidden) {
    extern __shared__ __align__(16) float side_shared[];       // [tokens][dim] gated values, [tokens][hidden] projected
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    float* gated = side_shared;
    float* projected = side_shared + SIDE_TOKENS * dim;
    const int t0 = blockIdx.x * SIDE_TOKENS;
    const int count = min(SIDE_TOKENS, n_tokens - t0);
    const float* rows[SIDE_TOKENS];
#pragma unroll
    for (int k = 0; k < SIDE_TOKENS; ++k) rows[k] = x + (size_t)(t0 + min(k, count - 1)) * hidden;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int j = warp; j < dim; j += warps) {
        const T* w_row = gate_w + (size_t)j * hidden;
        float dot[SIDE_TOKENS] = {};
        for (int c = lane; c < hidden; c += 32) {
            const float w = to_float(w_row[c]);
#pragma unroll
            for (int k = 0; k < SIDE_TOKENS; ++k) dot[k] = fmaf(w, rows[k][c], dot[k]);
        }
#pragma unroll
        for (int k = 0; k < SIDE_TOKENS; ++k) {
            const float total = warp_sum(dot[k]);
            if (lane == 0) {
                const int id = ids[t0 + min(k, count - 1)];
                // (the embedding has flagged an id outside the table)
                const bool known = id >= 0 && id < vocab;
                gated[k * dim + j] = known ? gelu_tanh(total) * to_float(table[(size_t)id * table_stride + offset + j]) : 0.0f;
            }
        }
    }
    __syncthreads();
    float partial[SIDE_TOKENS] = {};
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float sum[SIDE_TOKENS] = {};
        for (int j = 0; j < dim; ++j) {
            const float w = to_float(proj_t[(size_t)j * hidden + c]);
#pragma unroll
            for (int k = 0; k < SIDE_TOKENS; ++k) sum[k] = fmaf(w, gated[k * dim + j], sum[k]);
        }
#pragma unroll
        for (int k = 0; k < SIDE_TOKENS; ++k) {
            projected[(size_t)k * hidden + c] = sum[k];
            partial[k] = fmaf(sum[k], sum[k], partial[k]);
        }
    }
    float inverse_rms[SIDE_TOKENS];
#pragma unroll
    for (int k = 0; k < SIDE_TOKENS; ++k) inverse_rms[k] = 1.0f / sqrtf(block_sum(partial[k], scratch) / (float)hidden + eps);
    float squares[SIDE_TOKENS] = {};
    for (int k = 0; k < count; ++k) {
        float* x_row = x + (size_t)(t0 + k) * hidden;
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float v = x_row[c] + projected[(size_t)k * hidden + c] * inverse_rms[k] * norm_w[c];
            x_row[c] = v;
            squares[k] = fmaf(v, v, squares[k]);
        }
    }
    if (!next_out) return;
#pragma unroll
    for (int k = 0; k < SIDE_TOKENS; ++k) {
        const float next_inverse = 1.0f / sqrtf(block_sum(squares[k], scratch) / (float)hidden + next_eps);
        if (k >= count) continue;
        const float* x_row = x + (size_t)(t0 + k) * hidden;
        T* out_row = next_out + (size_t)(t0 + k) * hidden;
        for (int c = threadIdx.x; c < hidden; c += blockDim.x)     // (each thread reads back what it wrote itself)
            out_row[c] = from_float<T>(x_row[c] * next_inverse * next_gamma[c]);
    }
}

}  // namespace skv

using namespace skv;

static int stream_threads(int hidden) { return hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128); }

// x [n_rows, hidden] float += rmsnorm(y [n_rows, hidden] float) * gamma.  next_gamma and next_out (compute dtype,
// [n_rows, hidden]) both given: next_out = rmsnorm(new x) * next_gamma as well.
SKV_EXPORT int skv_rmsnorm_add(const float* y, const float* gamma, float eps, float* x, const float* next_gamma,
                               float next_eps, void* next_out, int n_rows, int hidden, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (hidden <= 0) return fail("skv_rmsnorm_add", "hidden must be positive");
    if ((next_gamma == nullptr) != (next_out == nullptr))
        return fail("skv_rmsnorm_add", "the next norm needs its weight and a place for its result");
    return launch_pdl("skv_rmsnorm_add", rmsnorm_add_kernel<skv_t>, dim3(n_rows), dim3(stream_threads(hidden)), 0,
                      stream, y, gamma, eps, x, next_gamma, next_eps, (skv_t*)next_out, hidden);
}

// table [vocab, table_stride], of whose rows the columns offset .. offset + dim - 1 are this layer's; gate_w
// [dim, hidden]; proj_t [dim, hidden], the projection transposed; norm_w float [hidden].
SKV_EXPORT int skv_token_side(float* x, const int* ids, const void* table, int table_stride, int offset, int dim,
                              int vocab, const void* gate_w, const void* proj_t, const float* norm_w, float eps,
                              const float* next_gamma, float next_eps, void* next_out, int n_tokens, int hidden,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || dim <= 0 || vocab <= 0) return fail("skv_token_side", "sizes must be positive");
    if (offset < 0 || offset + dim > table_stride) return fail("skv_token_side", "the layer's columns lie outside the table");
    if ((next_gamma == nullptr) != (next_out == nullptr))
        return fail("skv_token_side", "the next norm needs its weight and a place for its result");
    const size_t smem = (size_t)SIDE_TOKENS * (dim + hidden) * sizeof(float);
    if (smem > 200 * 1024) return fail("skv_token_side", "the stream is too wide for one block's shared memory");
    auto kernel = token_side_kernel<skv_t>;
    if (smem > 48 * 1024) {
        static bool raised = false;
        if (!raised) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
                return fail("skv_token_side", "cannot raise the shared-memory limit");
            raised = true;
        }
    }
    // few tokens: the blocks are few, so each is as large as it can be
    const int threads = n_tokens <= 64 * SIDE_TOKENS ? 1024 : stream_threads(hidden);
    return launch_pdl("skv_token_side", kernel, dim3((n_tokens + SIDE_TOKENS - 1) / SIDE_TOKENS), dim3(threads), smem,
                      stream, x, ids, (const skv_t*)table, table_stride, offset, dim, vocab, (const skv_t*)gate_w,
                      (const skv_t*)proj_t, norm_w, eps, next_gamma, next_eps, (skv_t*)next_out, n_tokens, hidden);
}
