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

// The same with the row held in registers (hidden a multiple of 4, at most 4 * VEC * blockDim, 16-byte aligned rows):
// a thread keeps VEC float4 of the branch and of the stream, so memory is read once and written once.
template <typename T, int VEC>
__global__ void rmsnorm_add_rows_kernel(const float* __restrict__ y, const float* __restrict__ gamma, float eps,
                                        float* __restrict__ x, const float* __restrict__ next_gamma, float next_eps,
                                        T* __restrict__ next_out, int hidden) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t r = blockIdx.x;
    const float4* y_row = (const float4*)(y + r * hidden);
    float4* x_row = (float4*)(x + r * hidden);
    const int quads = hidden >> 2;
    float4 branch[VEC], stream[VEC];
    float partial = 0.0f;
#pragma unroll
    for (int u = 0; u < VEC; ++u) {
        const int i = threadIdx.x + u * blockDim.x;
        if (i < quads) {
            branch[u] = y_row[i];
            stream[u] = x_row[i];
            partial += branch[u].x * branch[u].x + branch[u].y * branch[u].y + branch[u].z * branch[u].z + branch[u].w * branch[u].w;
        }
    }
    const float inverse_rms = 1.0f / sqrtf(block_sum(partial, scratch) / (float)hidden + eps);
    float squares = 0.0f;
#pragma unroll
    for (int u = 0; u < VEC; ++u) {
        const int i = threadIdx.x + u * blockDim.x;
        if (i < quads) {
            const float4 g = ((const float4*)gamma)[i];
            stream[u].x += branch[u].x * inverse_rms * g.x; stream[u].y += branch[u].y * inverse_rms * g.y;
            stream[u].z += branch[u].z * inverse_rms * g.z; stream[u].w += branch[u].w * inverse_rms * g.w;
            x_row[i] = stream[u];
            squares += stream[u].x * stream[u].x + stream[u].y * stream[u].y + stream[u].z * stream[u].z + stream[u].w * stream[u].w;
        }
    }
    if (!next_out) return;
    const float next_inverse = 1.0f / sqrtf(block_sum(squares, scratch) / (float)hidden + next_eps);
    T* out_row = next_out + r * hidden;
#pragma unroll
    for (int u = 0; u < VEC; ++u) {
        const int i = threadIdx.x + u * blockDim.x;
        if (i < quads) {
            const float4 g = ((const float4*)next_gamma)[i];
            out_row[4 * i] = from_float<T>(stream[u].x * next_inverse * g.x);
            out_row[4 * i + 1] = from_float<T>(stream[u].y * next_inverse * g.y);
            out_row[4 * i + 2] = from_float<T>(stream[u].z * next_inverse * g.z);
            out_row[4 * i + 3] = from_float<T>(stream[u].w * next_inverse * g.w);
        }
    }
}

// Four neighbouring weights of a row as floats (the row 8-byte aligned at `p` for bfloat16, 16-byte for float).
__device__ __forceinline__ void load4(const float* p, float (&out)[4]) {
    const float4 v = *(const float4*)p;
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&out)[4]) {
    const uint2 raw = *(const uint2*)p;
    const float2 lo = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x), hi = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
    out[0] = lo.x; out[1] = lo.y; out[2] = hi.x; out[3] = hi.y;
}

// A block takes TOK tokens, so that it reads the two weights once for all of them (one token a block where tokens are
// few, so that there are blocks enough).  `proj_t` is the projection transposed, [dim][hidden], which lets
// neighbouring threads read neighbouring columns.  VEC: hidden is a multiple of 4 and every row 16-byte aligned; a
// lane then takes four neighbouring columns at a time.  A warp works on four of the dim gate rows at once.
template <typename T, int TOK, bool VEC>
__global__ void __launch_bounds__(TOK == 1 ? 512 : 256) token_side_kernel(float* __restrict__ x, const int* __restrict__ ids, const T* __restrict__ table,
                                  int table_stride, int offset, int dim, int vocab, const T* __restrict__ gate_w,
                                  const T* __restrict__ proj_t, const float* __restrict__ norm_w, float eps,
                                  const float* __restrict__ next_gamma, float next_eps, T* __restrict__ next_out,
                                  int n_tokens, int hidden, const float* __restrict__ branch,
                                  const float* __restrict__ post_gamma, float post_eps) {
    extern __shared__ __align__(16) float side_shared[];       // [TOK][dim] gated values, [TOK][hidden] projected
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    float* gated = side_shared;
    float* projected = side_shared + TOK * ((dim + 3) & ~3);
    const int t0 = blockIdx.x * TOK;
    const int count = min(TOK, n_tokens - t0);
    const float* rows[TOK];
#pragma unroll
    for (int k = 0; k < TOK; ++k) rows[k] = x + (size_t)(t0 + min(k, count - 1)) * hidden;
    if (branch) {
        // first the sublayer in front: x += rmsnorm(branch) * post_gamma on this block's rows (rmsnorm_add's work)
#pragma unroll
        for (int k = 0; k < TOK; ++k) {
            const float* y_row = branch + (size_t)(t0 + min(k, count - 1)) * hidden;
            float sum = 0.0f;
            for (int c = threadIdx.x; c < hidden; c += blockDim.x) sum = fmaf(y_row[c], y_row[c], sum);
            const float inverse = 1.0f / sqrtf(block_sum(sum, scratch) / (float)hidden + post_eps);
            if (k < count) {
                float* x_row = x + (size_t)(t0 + k) * hidden;
                for (int c = threadIdx.x; c < hidden; c += blockDim.x) x_row[c] += y_row[c] * inverse * post_gamma[c];
            }
        }
        __syncthreads();                                       // (the rows are read by other threads from here on)
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    if (VEC) {
        // the block's rows of the stream go to shared memory once (the place of the projected values, which come
        // later), with every thread's loads in flight together; the gate rows then meet them there
        const int quads = hidden >> 2;
        for (int i = threadIdx.x; i < TOK * quads; i += blockDim.x) {
            const int k = i / quads, q4 = i - k * quads;
            ((float4*)projected)[i] = *(const float4*)(x + (size_t)(t0 + min(k, count - 1)) * hidden + 4 * q4);
        }
        __syncthreads();
    }
    for (int j0 = 4 * warp; j0 < dim; j0 += 4 * warps) {
        float dot[4][TOK] = {};
        const T* w_rows[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) w_rows[jj] = gate_w + (size_t)min(j0 + jj, dim - 1) * hidden;
        if (VEC) {
#pragma unroll 2
            for (int c = 4 * lane; c < hidden; c += 128) {
                float w[4][4];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) load4(w_rows[jj] + c, w[jj]);
#pragma unroll
                for (int k = 0; k < TOK; ++k) {
                    const float4 xs = *(const float4*)(projected + (size_t)k * hidden + c);
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj)
                        dot[jj][k] += w[jj][0] * xs.x + w[jj][1] * xs.y + w[jj][2] * xs.z + w[jj][3] * xs.w;
                }
            }
        } else {
            for (int c = lane; c < hidden; c += 32) {
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const float w = to_float(w_rows[jj][c]);
#pragma unroll
                    for (int k = 0; k < TOK; ++k) dot[jj][k] = fmaf(w, rows[k][c], dot[jj][k]);
                }
            }
        }
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
            for (int k = 0; k < TOK; ++k) {
                const float total = warp_sum(dot[jj][k]);
                if (lane == 0 && j0 + jj < dim) {
                    const int id = ids[t0 + min(k, count - 1)];
                    // (the embedding has flagged an id outside the table)
                    const bool known = id >= 0 && id < vocab;
                    gated[k * dim + j0 + jj] =
                        known ? gelu_tanh(total) * to_float(table[(size_t)id * table_stride + offset + j0 + jj]) : 0.0f;
                }
            }
        }
    }
    __syncthreads();
    float partial[TOK] = {};
    // four columns a thread at a time: a gated value is read from shared memory once for the four
    for (int c0 = threadIdx.x; c0 < hidden; c0 += 4 * blockDim.x) {
        float sum[4][TOK] = {};
        int cols[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) cols[i] = min(c0 + i * (int)blockDim.x, hidden - 1);
#pragma unroll 2
        for (int j = 0; j < dim; ++j) {
            float g[TOK];
#pragma unroll
            for (int k = 0; k < TOK; ++k) g[k] = gated[k * dim + j];
            const T* w_row = proj_t + (size_t)j * hidden;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float w = to_float(w_row[cols[i]]);
#pragma unroll
                for (int k = 0; k < TOK; ++k) sum[i][k] = fmaf(w, g[k], sum[i][k]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = c0 + i * (int)blockDim.x;
            if (c >= hidden) continue;
#pragma unroll
            for (int k = 0; k < TOK; ++k) {
                projected[(size_t)k * hidden + c] = sum[i][k];
                partial[k] = fmaf(sum[i][k], sum[i][k], partial[k]);
            }
        }
    }
    float inverse_rms[TOK];
#pragma unroll
    for (int k = 0; k < TOK; ++k) inverse_rms[k] = 1.0f / sqrtf(block_sum(partial[k], scratch) / (float)hidden + eps);
    float squares[TOK] = {};
#pragma unroll
    for (int k = 0; k < TOK; ++k) {
        if (k >= count) continue;
        float* x_row = x + (size_t)(t0 + k) * hidden;
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float v = x_row[c] + projected[(size_t)k * hidden + c] * inverse_rms[k] * norm_w[c];
            x_row[c] = v;
            squares[k] = fmaf(v, v, squares[k]);
        }
    }
    if (!next_out) return;
#pragma unroll
    for (int k = 0; k < TOK; ++k) {
        const float next_inverse = 1.0f / sqrtf(block_sum(squares[k], scratch) / (float)hidden + next_eps);
        if (k >= count) continue;
        const float* x_row = x + (size_t)(t0 + k) * hidden;
        T* out_row = next_out + (size_t)(t0 + k) * hidden;
        for (int c = threadIdx.x; c < hidden; c += blockDim.x)     // (each thread reads back what it wrote itself)
            out_row[c] = from_float<T>(x_row[c] * next_inverse * next_gamma[c]);
    }
}

template <int TOK, bool VEC>
static int launch_token_side(float* x, const int* ids, const void* table, int table_stride, int offset, int dim,
                             int vocab, const void* gate_w, const void* proj_t, const float* norm_w, float eps,
                             const float* next_gamma, float next_eps, void* next_out, int n_tokens, int hidden,
                             const float* branch, const float* post_gamma, float post_eps, int threads,
                             cudaStream_t stream) {
    const size_t smem = (size_t)TOK * (((dim + 3) & ~3) + hidden) * sizeof(float);
    auto kernel = token_side_kernel<skv_t, TOK, VEC>;
    if (smem > 48 * 1024) {
        static bool raised = false;
        if (!raised) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
                return fail("skv_token_side", "cannot raise the shared-memory limit");
            raised = true;
        }
    }
    return launch_pdl("skv_token_side", kernel, dim3((n_tokens + TOK - 1) / TOK), dim3(threads), smem, stream, x, ids,
                      (const skv_t*)table, table_stride, offset, dim, vocab, (const skv_t*)gate_w, (const skv_t*)proj_t,
                      norm_w, eps, next_gamma, next_eps, (skv_t*)next_out, n_tokens, hidden, branch, post_gamma, post_eps);
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
    const int threads = stream_threads(hidden);
    const bool aligned = hidden % 4 == 0 &&
                         (((uintptr_t)y | (uintptr_t)x | (uintptr_t)gamma | (uintptr_t)next_gamma) & 15) == 0;
    if (aligned && hidden <= 4 * 4 * threads)
        return launch_pdl("skv_rmsnorm_add", rmsnorm_add_rows_kernel<skv_t, 4>, dim3(n_rows), dim3(threads), 0, stream, y,
                          gamma, eps, x, next_gamma, next_eps, (skv_t*)next_out, hidden);
    return launch_pdl("skv_rmsnorm_add", rmsnorm_add_kernel<skv_t>, dim3(n_rows), dim3(threads), 0,
                      stream, y, gamma, eps, x, next_gamma, next_eps, (skv_t*)next_out, hidden);
}

// table [vocab, table_stride], of whose rows the columns offset .. offset + dim - 1 are this layer's; gate_w
// [dim, hidden]; proj_t [dim, hidden], the projection transposed; norm_w float [hidden].  branch and post_gamma
// (both or neither): x += rmsnorm(branch [n_tokens, hidden] float) * post_gamma comes first, in the same pass.
SKV_EXPORT int skv_token_side(float* x, const int* ids, const void* table, int table_stride, int offset, int dim,
                              int vocab, const void* gate_w, const void* proj_t, const float* norm_w, float eps,
                              const float* next_gamma, float next_eps, void* next_out, int n_tokens, int hidden,
                              const float* branch, const float* post_gamma, float post_eps, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || dim <= 0 || vocab <= 0) return fail("skv_token_side", "sizes must be positive");
    if ((branch == nullptr) != (post_gamma == nullptr))
        return fail("skv_token_side", "a branch needs the weight of the norm it passes on its way into the stream");
    if (offset < 0 || offset + dim > table_stride) return fail("skv_token_side", "the layer's columns lie outside the table");
    if ((next_gamma == nullptr) != (next_out == nullptr))
        return fail("skv_token_side", "the next norm needs its weight and a place for its result");
    if ((size_t)(((dim + 3) & ~3) + hidden) * sizeof(float) > 200 * 1024)
        return fail("skv_token_side", "the stream is too wide for one block's shared memory");
    const bool vec = hidden % 4 == 0 && (((uintptr_t)x | (uintptr_t)gate_w) & 15) == 0 && sizeof(skv_t) * hidden % 8 == 0;
    // eight tokens a block where their projected rows fit its shared memory, else four, else one; one token a block
    // where tokens are few, so that the step has blocks enough
    const size_t per_token = (size_t)(((dim + 3) & ~3) + hidden) * sizeof(float);
    const int tok = n_tokens <= 256 ? 1 : (8 * per_token <= 160 * 1024 ? 8 : (4 * per_token <= 200 * 1024 ? 4 : 1));
    const int threads = tok == 1 && hidden >= 1024 ? 512 : 256;      // (the many-token forms keep 100 to 200 registers a thread)
#define SKV_SIDE(TOK, VEC) launch_token_side<TOK, VEC>(x, ids, table, table_stride, offset, dim, vocab, gate_w, proj_t, norm_w, \
                                                      eps, next_gamma, next_eps, next_out, n_tokens, hidden, branch, post_gamma, \
                                                      post_eps, threads, stream)
    if (tok == 8) return vec ? SKV_SIDE(8, true) : SKV_SIDE(8, false);
    if (tok == 4) return vec ? SKV_SIDE(4, true) : SKV_SIDE(4, false);
    return vec ? SKV_SIDE(1, true) : SKV_SIDE(1, false);
#undef SKV_SIDE
}
