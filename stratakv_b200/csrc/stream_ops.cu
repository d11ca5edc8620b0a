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

template <typename T>
__global__ void token_side_kernel(float* __restrict__ x, const int* __restrict__ ids, const T* __restrict__ table,
                                  int table_stride, int offset, int dim, int vocab, const T* __restrict__ gate_w,
                                  const T* __restrict__ proj_w, const float* __restrict__ norm_w, float eps,
                                  const float* __restrict__ next_gamma, float next_eps, T* __restrict__ next_out,
                                  int hidden) {
    extern __shared__ __align__(16) float side_shared[];       // [dim] gated values, [hidden] projected values
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    float* gated = side_shared;
    float* projected = side_shared + dim;
    const size_t t = blockIdx.x;
    float* x_row = x + t * hidden;
    const int id = ids[t];
    const bool known = id >= 0 && id < vocab;                  // (the embedding has flagged an id outside the table)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int j = warp; j < dim; j += warps) {
        const T* w_row = gate_w + (size_t)j * hidden;
        float dot = 0.0f;
        for (int c = lane; c < hidden; c += 32) dot = fmaf(to_float(w_row[c]), x_row[c], dot);
        dot = warp_sum(dot);
        if (lane == 0) gated[j] = known ? gelu_tanh(dot) * to_float(table[(size_t)id * table_stride + offset + j]) : 0.0f;
    }
    __syncthreads();
    float partial = 0.0f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const T* w_row = proj_w + (size_t)c * dim;
        float sum = 0.0f;
        for (int j = 0; j < dim; ++j) sum = fmaf(to_float(w_row[j]), gated[j], sum);
        projected[c] = sum;
        partial = fmaf(sum, sum, partial);
    }
    const float inverse_rms = 1.0f / sqrtf(block_sum(partial, scratch) / (float)hidden + eps);
    float squares = 0.0f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = x_row[c] + projected[c] * inverse_rms * norm_w[c];
        x_row[c] = v;
        squares = fmaf(v, v, squares);
    }
    if (!next_out) return;
    const float next_inverse = 1.0f / sqrtf(block_sum(squares, scratch) / (float)hidden + next_eps);
    T* out_row = next_out + t * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        out_row[c] = from_float<T>(x_row[c] * next_inverse * next_gamma[c]);
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
// [dim, hidden]; proj_w [hidden, dim]; norm_w float [hidden].
SKV_EXPORT int skv_token_side(float* x, const int* ids, const void* table, int table_stride, int offset, int dim,
                              int vocab, const void* gate_w, const void* proj_w, const float* norm_w, float eps,
                              const float* next_gamma, float next_eps, void* next_out, int n_tokens, int hidden,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || dim <= 0 || vocab <= 0) return fail("skv_token_side", "sizes must be positive");
    if (offset < 0 || offset + dim > table_stride) return fail("skv_token_side", "the layer's columns lie outside the table");
    if ((next_gamma == nullptr) != (next_out == nullptr))
        return fail("skv_token_side", "the next norm needs its weight and a place for its result");
    const size_t smem = (size_t)(dim + hidden) * sizeof(float);
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
    return launch_pdl("skv_token_side", kernel, dim3(n_tokens), dim3(stream_threads(hidden)), smem, stream, x, ids,
                      (const skv_t*)table, table_stride, offset, dim, vocab, (const skv_t*)gate_w, (const skv_t*)proj_w,
                      norm_w, eps, next_gamma, next_eps, (skv_t*)next_out, hidden);
}
