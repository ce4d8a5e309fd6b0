// Pre-norm layers on a residual stream that is kept in 32-bit whatever the activation dtype.
//
//   embed_norm      : x[t] = N(table[id_t]) * w                     (the stream's first value; table rows are activations)
//   stream_add_norm : v = x + s * y   (s: a scale per channel, or none; without y: v = x; with `unit_eps` >= 0 y is
//                     first divided by its root mean square, sqrt(mean(y^2) + unit_eps))
//                     x_out = v (may be x itself), h = N(v) * w rounded to the activation dtype (what the next
//                     sublayer's products read; N may be "none": h is v rounded)
//   stream_add_many : v = x + sum_i s_i * y_i (up to four addends, a scalar each), x_out = v in place, h = N(v) * w
//   stream_pair_rows: [x rounded | x0] side by side, the input of a product over the stream and the rows it began as
//   side_gate       : a = gelu_tanh(z) * e for the products z [tokens, dim] of a side input's gate (see below), for
//                     steps of many tokens, whose two small products go to the library
//   stream_side     : v = x + s * y as above, then the token's side input
//                       a = gelu_tanh(G v) * e      (G [dim, H]; e: `dim` columns of the token's row of a side table)
//                       u = P a                     (P [H, dim], handed over transposed)
//                       v <- v + u / sqrt(mean(u^2) + eps) * w_side
//                     x_out = v, and, when a norm follows at once, h = N(v) * w_next
//
// N is a layer norm without bias ((v - mean) / sqrt(var + eps), var the mean of the squared deviations, both passes
// over the row held in shared memory) or an RMS norm.  Sums, norms and the stream are float32; G, P and the tables
// are read in the dtype they are held in and multiplied in float32.
#include "lb200/common.cuh"
using namespace lb200;

enum : int { kLayerNorm = 0, kRmsNorm = 1, kNoNorm = 2 };

// 1 / sqrt(var + eps) and the mean of the row in shared memory (`row`, H floats); all threads get both
__device__ __forceinline__ void row_stats(const float* row, int H, int kind, float eps, float* red, float& mean, float& inv) {
    mean = 0.f;
    if (kind == kNoNorm) { inv = 1.f; return; }
    if (kind == kLayerNorm) {
        float s = 0.f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) s += row[c];
        mean = block_sum(s, red) / (float)H;
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float d = row[c] - mean;
        ss += d * d;
    }
    inv = 1.f / sqrtf(block_sum(ss, red) / (float)H + eps);
}

template <typename T>
__global__ void embed_norm_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                  const float* __restrict__ w, float eps, int H, int V, int kind, int* bad_ids) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const size_t t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && bad_ids) atomicAdd(bad_ids, 1);
        id = min(max(id, 0), V - 1);
    }
    const T* src = table + (size_t)id * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) row[c] = to_f32(src[c]);
    __syncthreads();
    float mean, inv;
    row_stats(row, H, kind, eps, red, mean, inv);
    for (int c = threadIdx.x; c < H; c += blockDim.x) out[t * H + c] = (row[c] - mean) * inv * w[c];
}

extern "C" int lb_embed_norm(float* out, const void* table, const int* ids, const float* w, float eps, int tokens, int H, int V,
                             int kind, int* bad_ids, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (H <= 0 || V <= 0 || (size_t)H * sizeof(float) > 160 * 1024 || (kind != kLayerNorm && kind != kRmsNorm)) return kBadSize;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const size_t smem = (size_t)H * sizeof(float);
    LB_DISPATCH_DTYPE(dtype, {
        static size_t have = 0;
        ensure_dynamic_smem(embed_norm_kernel<T>, smem, have);
        embed_norm_kernel<T><<<tokens, threads, smem, (cudaStream_t)stream>>>(out, (const T*)table, ids, w, eps, H, V, kind, bad_ids);
    });
    return launch_status();
}

template <typename T>
__global__ void stream_add_norm_kernel(const float* x, const T* __restrict__ y, const float* __restrict__ ls, float unit_eps,
                                       const float* __restrict__ w, float eps, float* x_out, T* __restrict__ h_out, int H, int kind) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
    float y_scale = 1.f;
    if (y != nullptr && unit_eps >= 0.f) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) { const float v = to_f32(y[base + c]); ss += v * v; }
        y_scale = 1.f / sqrtf(block_sum(ss, red) / (float)H + unit_eps);
    }
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = x[base + c];
        if (y != nullptr) v += (ls != nullptr ? ls[c] : 1.f) * y_scale * to_f32(y[base + c]);
        row[c] = v;
        if (x_out != nullptr) x_out[base + c] = v;
    }
    if (h_out == nullptr) return;
    __syncthreads();
    float mean, inv;
    row_stats(row, H, kind, eps, red, mean, inv);
    for (int c = threadIdx.x; c < H; c += blockDim.x) h_out[base + c] = from_f32<T>((row[c] - mean) * inv * (w != nullptr ? w[c] : 1.f));
}

extern "C" int lb_stream_add_norm(const float* x, const void* y, const float* ls, float unit_eps, const float* w, float eps,
                                  float* x_out, void* h_out, int rows, int H, int kind, int dtype, void* stream) {
    if (rows <= 0) return kOk;
    if (H <= 0 || (size_t)H * sizeof(float) > 160 * 1024 || kind < kLayerNorm || kind > kNoNorm) return kBadSize;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const size_t smem = (size_t)H * sizeof(float);
    LB_DISPATCH_DTYPE(dtype, {
        static size_t have = 0;
        ensure_dynamic_smem(stream_add_norm_kernel<T>, smem, have);
        stream_add_norm_kernel<T><<<rows, threads, smem, (cudaStream_t)stream>>>(x, (const T*)y, ls, unit_eps, w, eps, x_out, (T*)h_out, H, kind);
    });
    return launch_status();
}

// v = x + sum_i s_i * y_i for up to four addends with a scalar each (the sublayers of a block whose mixers and feed-forward all
// read one norm's output), x_out = v in place, h = N(v) * w as in `stream_add_norm`
struct Addends {
    const void* y[4];
    float s[4];
    int n;
};

template <typename T>
__global__ void stream_add_many_kernel(float* x, Addends a, const float* __restrict__ w, float eps, T* __restrict__ h_out, int H, int kind) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = x[base + c];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (i < a.n) v += a.s[i] * to_f32(((const T*)a.y[i])[base + c]);
        row[c] = v;
        x[base + c] = v;
    }
    if (h_out == nullptr) return;
    __syncthreads();
    float mean, inv;
    row_stats(row, H, kind, eps, red, mean, inv);
    for (int c = threadIdx.x; c < H; c += blockDim.x) h_out[base + c] = from_f32<T>((row[c] - mean) * inv * (w != nullptr ? w[c] : 1.f));
}

extern "C" int lb_stream_add_many(float* x, const void* y0, const void* y1, const void* y2, const void* y3, float s0, float s1, float s2,
                                  float s3, int n, const float* w, float eps, void* h_out, int rows, int H, int kind, int dtype,
                                  void* stream) {
    if (rows <= 0) return kOk;
    if (H <= 0 || (size_t)H * sizeof(float) > 160 * 1024 || kind < kLayerNorm || kind > kNoNorm || n < 0 || n > 4) return kBadSize;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const size_t smem = (size_t)H * sizeof(float);
    const Addends a = {{y0, y1, y2, y3}, {s0, s1, s2, s3}, n};
    LB_DISPATCH_DTYPE(dtype, {
        static size_t have = 0;
        ensure_dynamic_smem(stream_add_many_kernel<T>, smem, have);
        stream_add_many_kernel<T><<<rows, threads, smem, (cudaStream_t)stream>>>(x, a, w, eps, (T*)h_out, H, kind);
    });
    return launch_status();
}

// out[t] = [x[t] rounded to the activation dtype | x0[t]]: the input of a product that mixes the stream with the rows it began as
template <typename T>
__global__ void stream_pair_rows_kernel(const float* __restrict__ x, const T* __restrict__ x0, T* __restrict__ out, int H, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / (2 * H);
    const int c = (int)(i % (2 * H));
    out[i] = c < H ? from_f32<T>(x[t * H + c]) : x0[t * H + (c - H)];
}

extern "C" int lb_stream_pair_rows(const float* x, const void* x0, void* out, int rows, int H, int dtype, void* stream) {
    if (rows <= 0) return kOk;
    if (H <= 0) return kBadSize;
    const size_t total = (size_t)rows * 2 * H;
    LB_DISPATCH_DTYPE(dtype, stream_pair_rows_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        x, (const T*)x0, (T*)out, H, total));
    return launch_status();
}

// z, a: [tokens, dim]
template <typename T>
__global__ void side_gate_kernel(const T* __restrict__ z, const int* __restrict__ ids, const T* __restrict__ side_table, int table_width,
                                 int offset, int V, T* __restrict__ a, int dim, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / dim;
    const int d = (int)(i % dim);
    const int id = min(max(ids[t], 0), V - 1);
    const float v = to_f32(z[i]);
    a[i] = from_f32<T>(0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)))
                       * to_f32(side_table[(size_t)id * table_width + offset + d]));
}

extern "C" int lb_side_gate(const void* z, const int* ids, const void* side_table, int table_width, int offset, int V, void* a,
                            int tokens, int dim, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (dim <= 0 || offset < 0 || offset + dim > table_width || V <= 0) return kBadSize;
    const size_t total = (size_t)tokens * dim;
    LB_DISPATCH_DTYPE(dtype, side_gate_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (const T*)z, ids, (const T*)side_table, table_width, offset, V, (T*)a, dim, total));
    return launch_status();
}

// Sums of `kTok` values over a whole block at once; `scratch` is >= 32 * kTok floats.  All threads get the results.
template <int kTok>
__device__ __forceinline__ void block_sum_multi(float (&v)[kTok], float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int k = 0; k < kTok; ++k) v[k] = warp_sum(v[k]);
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < kTok; ++k) scratch[k * 32 + warp] = v[k];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kTok; ++k) v[k] = warp_sum(lane < nwarps ? scratch[k * 32 + lane] : 0.f);
}

// grid (ceil(tokens / kTok)): a CTA takes kTok neighbouring tokens, so that the two small matrices are read once for
// all of them; shared memory: rows [kTok][H] | a [kTok][dim].  proj_t is P transposed, [dim, H] (columns of a token's
// output lie side by side).  u = P a is computed twice (for its mean square, then for the sum) instead of being kept.
template <typename T, int kTok>
__global__ void stream_side_kernel(const float* x, const T* __restrict__ y, const float* __restrict__ ls,
                                   const int* __restrict__ ids, const T* __restrict__ side_table, int table_width, int offset,
                                   int V, const T* __restrict__ gate_w, const T* __restrict__ proj_t,
                                   const float* __restrict__ side_w, float side_eps, int dim, const float* __restrict__ next_w,
                                   float next_eps, int next_kind, float* x_out, T* __restrict__ h_out, int H, int tokens) {
    extern __shared__ float smem[];
    __shared__ float red[32 * kTok];
    float* rows = smem;                    // [kTok][H]
    float* a = smem + (size_t)kTok * H;    // [kTok][dim]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int t0 = blockIdx.x * kTok;
    const int n = min(kTok, tokens - t0);
#pragma unroll
    for (int k = 0; k < kTok; ++k) {
        const size_t base = (size_t)(t0 + k) * H;
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float v = 0.f;
            if (k < n) {
                v = x[base + c];
                if (y != nullptr) v += (ls != nullptr ? ls[c] : 1.f) * to_f32(y[base + c]);
            }
            rows[k * H + c] = v;
        }
    }
    __syncthreads();
    for (int d = warp; d < dim; d += nwarps) {
        const T* g = gate_w + (size_t)d * H;
        float acc[kTok];
#pragma unroll
        for (int k = 0; k < kTok; ++k) acc[k] = 0.f;
#pragma unroll 4
        for (int c = lane; c < H; c += 32) {
            const float w = to_f32(g[c]);
#pragma unroll
            for (int k = 0; k < kTok; ++k) acc[k] += w * rows[k * H + c];
        }
#pragma unroll
        for (int k = 0; k < kTok; ++k) {
            const float z = warp_sum(acc[k]);
            if (lane == 0 && k < n) {
                const int id = min(max(ids[t0 + k], 0), V - 1);
                const float e = to_f32(side_table[(size_t)id * table_width + offset + d]);
                a[k * dim + d] = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))) * e;
            } else if (lane == 0) {
                a[k * dim + d] = 0.f;
            }
        }
    }
    __syncthreads();
    float ss[kTok];
#pragma unroll
    for (int k = 0; k < kTok; ++k) ss[k] = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float u[kTok];
#pragma unroll
        for (int k = 0; k < kTok; ++k) u[k] = 0.f;
#pragma unroll 8
        for (int d = 0; d < dim; ++d) {
            const float w = to_f32(proj_t[(size_t)d * H + c]);
#pragma unroll
            for (int k = 0; k < kTok; ++k) u[k] += w * a[k * dim + d];
        }
#pragma unroll
        for (int k = 0; k < kTok; ++k) ss[k] += u[k] * u[k];
    }
    block_sum_multi<kTok>(ss, red);
    float inv_u[kTok];
#pragma unroll
    for (int k = 0; k < kTok; ++k) inv_u[k] = 1.f / sqrtf(ss[k] / (float)H + side_eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float u[kTok];
#pragma unroll
        for (int k = 0; k < kTok; ++k) u[k] = 0.f;
#pragma unroll 8
        for (int d = 0; d < dim; ++d) {
            const float w = to_f32(proj_t[(size_t)d * H + c]);
#pragma unroll
            for (int k = 0; k < kTok; ++k) u[k] += w * a[k * dim + d];
        }
        const float sw = side_w[c];
#pragma unroll
        for (int k = 0; k < kTok; ++k) {
            const float v = rows[k * H + c] + u[k] * inv_u[k] * sw;
            rows[k * H + c] = v;                       // (this thread's own column: no other thread reads it before the barrier below)
            if (k < n) x_out[(size_t)(t0 + k) * H + c] = v;
        }
    }
    if (h_out == nullptr) return;
    float mean[kTok], var[kTok];
#pragma unroll
    for (int k = 0; k < kTok; ++k) mean[k] = 0.f;
    if (next_kind == kLayerNorm) {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
#pragma unroll
            for (int k = 0; k < kTok; ++k) mean[k] += rows[k * H + c];
        }
        block_sum_multi<kTok>(mean, red);
#pragma unroll
        for (int k = 0; k < kTok; ++k) mean[k] /= (float)H;
    }
#pragma unroll
    for (int k = 0; k < kTok; ++k) var[k] = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
#pragma unroll
        for (int k = 0; k < kTok; ++k) { const float dd = rows[k * H + c] - mean[k]; var[k] += dd * dd; }
    }
    block_sum_multi<kTok>(var, red);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float w = next_w[c];
#pragma unroll
        for (int k = 0; k < kTok; ++k)
            if (k < n) h_out[(size_t)(t0 + k) * H + c] = from_f32<T>((rows[k * H + c] - mean[k]) / sqrtf(var[k] / (float)H + next_eps) * w);
    }
}

template <typename T, int kTok>
static int launch_side(const float* x, const void* y, const float* ls, const int* ids, const void* side_table, int table_width,
                       int offset, int V, const void* gate_w, const void* proj_t, const float* side_w, float side_eps, int dim,
                       const float* next_w, float next_eps, int next_kind, float* x_out, void* h_out, int rows, int H, void* stream) {
    const size_t smem = ((size_t)kTok * H + (size_t)kTok * dim) * sizeof(float);
    static size_t have = 0;
    ensure_dynamic_smem(stream_side_kernel<T, kTok>, smem, have);
    // one token per CTA means few CTAs (a decode step): more warps each, so that more loads of the matrices are in flight
    const int threads = kTok == 1 ? (H >= 1024 ? 1024 : 512) : (H >= 2048 ? 512 : 256);
    stream_side_kernel<T, kTok><<<(rows + kTok - 1) / kTok, threads, smem, (cudaStream_t)stream>>>(
        x, (const T*)y, ls, ids, (const T*)side_table, table_width, offset, V, (const T*)gate_w, (const T*)proj_t, side_w, side_eps,
        dim, next_w, next_eps, next_kind, x_out, (T*)h_out, H, rows);
    return launch_status();
}

extern "C" int lb_stream_side(const float* x, const void* y, const float* ls, const int* ids, const void* side_table,
                              int table_width, int offset, int V, const void* gate_w, const void* proj_t, const float* side_w,
                              float side_eps, int dim, const float* next_w, float next_eps, int next_kind, float* x_out,
                              void* h_out, int rows, int H, int dtype, void* stream) {
    if (rows <= 0) return kOk;
    if (H <= 0 || dim <= 0 || offset < 0 || offset + dim > table_width || V <= 0) return kBadSize;
    if (h_out != nullptr && next_kind != kLayerNorm && next_kind != kRmsNorm) return kBadSize;
    // tokens per CTA: as many as fit 96 KB of rows, fewer where the step has too few tokens to fill the GPU otherwise
    const size_t per_token = ((size_t)H + dim) * sizeof(float);
    if (per_token > 200 * 1024) return kTooLarge;
    int tok = 1;
    while (tok < 8 && (size_t)(2 * tok) * per_token <= 96 * 1024 && rows >= 148 * 2 * tok) tok *= 2;
#define LB_SIDE(TOK) LB_DISPATCH_DTYPE(dtype, return (launch_side<T, TOK>(x, y, ls, ids, side_table, table_width, offset, V, gate_w, proj_t, \
        side_w, side_eps, dim, next_w, next_eps, next_kind, x_out, h_out, rows, H, stream)))
    if (tok == 8) { LB_SIDE(8); }
    if (tok == 4) { LB_SIDE(4); }
    if (tok == 2) { LB_SIDE(2); }
    LB_SIDE(1);
#undef LB_SIDE
    return kBadDType;
}
