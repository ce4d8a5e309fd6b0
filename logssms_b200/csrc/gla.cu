// Gated linear attention with a decay per key channel, token by token.
//
//   a_t[d]  = sigmoid(z_t[d]) ^ (1 / tau)            (32-bit: log-sigmoid, division by tau, exponential)
//             or, with `head_decay`, one fixed decay per head for all its key channels and tokens (z is not read)
//   S_t     = diag(a_t) S_{t-1} + k_t v_t^T            (S: [key channels, value channels] per head, 32-bit)
//   o_t     = S_t^T (q_t * q_scale)
//
//  gla_scan      : the recurrence over every request's tokens of a step, state read from and written back to the
//                  request's slot (a request that starts at position 0 starts from zeros whatever the slot holds).
//                  A CTA owns (request, head, a tile of value channels); a thread owns R state rows of one value
//                  column, DS threads of a warp share a column.  q, k, the decays and v of 8 tokens at a time are
//                  staged in shared memory, so the inner loop touches registers and shared memory only.
//  gla_norm_gate : y = o / sqrt(mean_head(o^2) + eps) * w[c] * act(g), o in 32-bit, w shared by the heads; act is
//                  silu or the sigmoid.  With one "head" of the full width it is the gated norm over all heads together.
#include "lb200/common.cuh"
using namespace lb200;

constexpr int kGlaTokens = 8;

__device__ __forceinline__ float log_sigmoid(float z) {
    return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z));
}

template <typename T, int R, int DS>
__global__ void gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long row_stride,
                                const float* __restrict__ z, float* __restrict__ o, float* state,
                                const int* __restrict__ cu, const int* __restrict__ start_pos, const int* __restrict__ slots,
                                const int* __restrict__ request_list, int H, int dim, int vdim, float inv_tau, float q_scale,
                                const float* __restrict__ head_decay) {
    constexpr int DP = R * DS;                       // key channels, padded
    extern __shared__ float sm[];
    const int cols = blockDim.x / DS;
    float* qs = sm;                                  // [kGlaTokens][DP]
    float* ks = qs + kGlaTokens * DP;
    float* as = ks + kGlaTokens * DP;
    float* vs = as + kGlaTokens * DP;                // [kGlaTokens][cols]
    const int b = request_list ? request_list[blockIdx.z] : blockIdx.z;
    if (b < 0) return;
    const int h = blockIdx.y;
    const int col_local = threadIdx.x / DS, s = threadIdx.x % DS;
    const int c = blockIdx.x * cols + col_local;
    const int first = cu[b], last = cu[b + 1];
    const size_t sbase = ((size_t)slots[b] * H + h) * dim * vdim;
    const bool fresh = start_pos[b] == 0;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = s * R + r;
        S[r] = (!fresh && d < dim && c < vdim) ? state[sbase + (size_t)d * vdim + c] : 0.f;
    }
    for (int t0 = first; t0 < last; t0 += kGlaTokens) {
        const int n = min(kGlaTokens, last - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < n * DP; i += blockDim.x) {
            const int tt = i / DP, d = i % DP;
            float qv = 0.f, kv = 0.f, av = 0.f;
            if (d < dim) {
                const size_t row = (size_t)(t0 + tt);
                qv = to_f32(q[row * row_stride + h * dim + d]) * q_scale;
                kv = to_f32(k[row * row_stride + h * dim + d]);
                av = head_decay != nullptr ? head_decay[h] : expf(log_sigmoid(z[(row * H + h) * dim + d]) * inv_tau);
            }
            qs[i] = qv; ks[i] = kv; as[i] = av;
        }
        for (int i = threadIdx.x; i < n * cols; i += blockDim.x) {
            const int tt = i / cols, cc = blockIdx.x * cols + i % cols;
            vs[i] = cc < vdim ? to_f32(v[(size_t)(t0 + tt) * row_stride + h * vdim + cc]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float vv = vs[tt * cols + col_local];
            const float* qr = qs + tt * DP + s * R;
            const float* kr = ks + tt * DP + s * R;
            const float* ar = as + tt * DP + s * R;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                S[r] = ar[r] * S[r] + kr[r] * vv;
                acc += qr[r] * S[r];
            }
#pragma unroll
            for (int off = 1; off < DS; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (s == 0 && c < vdim) o[((size_t)(t0 + tt) * H + h) * vdim + c] = acc;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = s * R + r;
        if (d < dim && c < vdim) state[sbase + (size_t)d * vdim + c] = S[r];
    }
}

template <typename T, int R, int DS>
static int launch_gla_scan(const void* q, const void* k, const void* v, long row_stride, const float* z, float* o, float* state,
                           const int* cu, const int* start_pos, const int* slots, const int* request_list, int num_requests,
                           int H, int dim, int vdim, float inv_tau, float q_scale, const float* head_decay, cudaStream_t stream) {
    // few requests: narrow tiles, so that more CTAs share the work
    const int want = (num_requests * H * ((vdim * DS + 127) / 128) < 148) ? 32 : 128;
    const int threads = min(want, (vdim * DS + 31) / 32 * 32);
    const int cols = threads / DS;
    dim3 grid((vdim + cols - 1) / cols, H, num_requests);
    const size_t smem = (size_t)kGlaTokens * (3 * R * DS + cols) * sizeof(float);
    static size_t have = 0;
    ensure_dynamic_smem(gla_scan_kernel<T, R, DS>, smem, have);
    gla_scan_kernel<T, R, DS><<<grid, threads, smem, stream>>>((const T*)q, (const T*)k, (const T*)v, row_stride, z, o, state, cu,
                                                               start_pos, slots, request_list, H, dim, vdim, inv_tau, q_scale, head_decay);
    return launch_status();
}

// q, k: [tokens, H*dim] and v: [tokens, H*vdim], column views of one projection buffer (common row stride, in
// elements); z: float32 [tokens, H*dim]; o: float32 [tokens, H*vdim]; state: float32 [slots, H, dim, vdim].
extern "C" int lb_gla_scan(const void* q, const void* k, const void* v, long row_stride, const float* z, float* o, float* state,
                           const int* cu, const int* start_pos, const int* slots, const int* request_list, int num_requests,
                           int H, int dim, int vdim, float tau, float q_scale, const float* head_decay, int dtype, void* stream) {
    if (num_requests <= 0) return kOk;
    if (H <= 0 || dim <= 0 || vdim <= 0 || !(tau > 0.f)) return kBadSize;
    if (dim > 512) return kTooLarge;
    cudaStream_t st = (cudaStream_t)stream;
#define LB_GLA(R_, DS_) LB_DISPATCH_DTYPE(dtype, return (launch_gla_scan<T, R_, DS_>(q, k, v, row_stride, z, o, state, cu, start_pos, \
        slots, request_list, num_requests, H, dim, vdim, 1.f / tau, q_scale, head_decay, st)))
    if (dim <= 16) { LB_GLA(16, 1); }
    else if (dim <= 32) { LB_GLA(32, 1); }
    else if (dim <= 64) { LB_GLA(64, 1); }
    else if (dim <= 128) { LB_GLA(64, 2); }
    else if (dim <= 256) { LB_GLA(64, 4); }
    else { LB_GLA(64, 8); }
#undef LB_GLA
    return kOk;
}

// grid (rows, heads)
template <typename T>
__global__ void gla_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, long gate_stride,
                                     const float* __restrict__ weight, T* __restrict__ out, int H, int vdim, float eps,
                                     int sigmoid_gate) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const int h = blockIdx.y;
    const float* orow = o + (row * H + h) * vdim;
    float ss = 0.f;
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) ss += orow[c] * orow[c];
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)vdim + eps);
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
        const float g = to_f32(gate[row * gate_stride + h * vdim + c]);
        out[(row * H + h) * vdim + c] = from_f32<T>(orow[c] * inv * weight[c] * (sigmoid_gate ? 1.f / (1.f + expf(-g)) : silu_f(g)));
    }
}

extern "C" int lb_gla_norm_gate(const float* o, const void* gate, long gate_stride, const float* weight, void* out, int rows,
                                int H, int vdim, float eps, int sigmoid_gate, int dtype, void* stream) {
    if (rows <= 0) return kOk;
    if (H <= 0 || vdim <= 0 || H > 65535) return kBadSize;
    const int threads = min(256, (vdim + 31) / 32 * 32);
    dim3 grid(rows, H);
    LB_DISPATCH_DTYPE(dtype, gla_norm_gate_kernel<T><<<grid, threads, 0, (cudaStream_t)stream>>>(
        o, (const T*)gate, gate_stride, weight, (T*)out, H, vdim, eps, sigmoid_gate));
    return launch_status();
}

// ------------------------------------------------------------------------------------------------------------------
// Prompt portions in chunks of 16 tokens (bfloat16 engines).  With b_i[d] the running sum of the log-decays inside a
// chunk (inclusive), a chunk that starts from the state S_in gives
//     o_i   = (q_i * e^{b_i}) S_in  +  sum_{j <= i} A_ij v_j ,     A_ij = sum_d q_i[d] k_j[d] e^{b_i[d] - b_j[d]}
//     S_out = diag(e^{b_end}) S_in  +  sum_j (k_j * e^{b_end - b_j}) v_j^T
// and every exponent is <= 0, whatever the decays are: nothing can overflow, and what underflows is truly nothing.
//
//  gla_chunk_prepare : one CTA per (chunk, head), all chunks of a step side by side: log-decays and their running sums
//                      in 32-bit, A in 32-bit (a thread per pair and key-channel slice), the scaled operands
//                      q * e^{b} and k * e^{b_end - b} rounded to bfloat16 for the tensor cores, e^{b_end} in 32-bit.
//  gla_chunk_scan    : one CTA per (request, head, 32 value columns) walks the request's chunks in order.  The state
//                      lives in 32-bit in the accumulator registers of `mma.sync` tiles (rows: key channels) from the
//                      slot to the slot; per chunk it is scaled by e^{b_end}, takes (k e^{..})^T v on the tensor
//                      cores, and a bfloat16 copy of it in shared memory is the operand of (q e^{b}) S_in.  The
//                      chunk's own A v is added in 32-bit.
constexpr int kChunk = 16;
constexpr int kScanCols = 32;

__global__ void __launch_bounds__(128) gla_chunk_prepare_kernel(
        const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, long row_stride, const float* __restrict__ z,
        const int* __restrict__ cu, const int* __restrict__ chunks, __nv_bfloat16* __restrict__ q_in,
        __nv_bfloat16* __restrict__ k_end, float* __restrict__ A, float* __restrict__ D, int H, int dim, float inv_tau,
        float q_scale, const float* __restrict__ head_decay) {
    extern __shared__ float sm[];
    float* b = sm;                         // [16][dim] log-decays, then their running sums
    float* qs = b + kChunk * dim;
    float* ks = qs + kChunk * dim;
    const int c = blockIdx.x, h = blockIdx.y;
    const int req = chunks[2 * c];
    if (req < 0) return;
    const int t0 = cu[req] + chunks[2 * c + 1];
    const int n = min(kChunk, cu[req + 1] - t0);
    for (int i = threadIdx.x; i < kChunk * dim; i += blockDim.x) {
        const int j = i / dim, d = i % dim;
        float ld = 0.f, qv = 0.f, kv = 0.f;
        if (j < n) {
            const size_t row = (size_t)(t0 + j);
            ld = head_decay != nullptr ? logf(head_decay[h]) : log_sigmoid(z[(row * H + h) * dim + d]) * inv_tau;
            qv = to_f32(q[row * row_stride + h * dim + d]) * q_scale;
            kv = to_f32(k[row * row_stride + h * dim + d]);
        }
        b[i] = ld; qs[i] = qv; ks[i] = kv;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < kChunk; ++j) { acc += b[j * dim + d]; b[j * dim + d] = acc; }
        D[((size_t)c * H + h) * dim + d] = expf(acc);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n * dim; i += blockDim.x) {
        const int j = i / dim, d = i % dim;
        const size_t at = ((size_t)(t0 + j) * H + h) * dim + d;
        q_in[at] = __float2bfloat16_rn(qs[i] * expf(b[i]));
        k_end[at] = __float2bfloat16_rn(ks[i] * expf(b[(kChunk - 1) * dim + d] - b[i]));
    }
    // A: a warp per pair (i, j), its lanes over the key channels
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int p = warp; p < n * kChunk; p += nwarps) {
        const int i = p / kChunk, j = p % kChunk;
        float a = 0.f;
        if (j <= i) {
            for (int d = lane; d < dim; d += 32) a += qs[i * dim + d] * ks[j * dim + d] * __expf(b[i * dim + d] - b[j * dim + d]);
            a = warp_sum(a);
        }
        if (lane == 0) A[((size_t)(t0 + i) * H + h) * kChunk + j] = a;
    }
}

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(__nv_bfloat16 lo, __nv_bfloat16 hi) {
    return (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
}

// grid (ceil(vdim / 32), H, work items); 4 warps; MT: 16-row state tiles per warp (dim <= 64 * MT).
// MODE 0: an item is a request (request, first chunk, chunks): from its slot's state to its slot's state, writing o.
// A lone long prompt has too few such items to fill the GPU, so it may run in segments of chunks instead, an item
// being (request, first chunk, chunks, first token within the portion):
// MODE 1: a segment from a zero state, no output: leaves its end state in seg_state[item] and the product of its
//         chunks' decays in seg_decay[item]; `gla_segment_pass` then turns the end states into start states;
// MODE 2: a segment from seg_state[item], writing o.
template <int MT, int MODE>
__global__ void __launch_bounds__(128) gla_chunk_scan_kernel(
        const __nv_bfloat16* __restrict__ q_in, const __nv_bfloat16* __restrict__ k_end, const __nv_bfloat16* __restrict__ v,
        long v_stride, const float* __restrict__ A, const float* __restrict__ D, float* __restrict__ o, float* state,
        const int* __restrict__ cu, const int* __restrict__ start_pos, const int* __restrict__ slots,
        const int* __restrict__ per_request, int H, int dim, int vdim, float* seg_state, float* seg_decay) {
    constexpr int NT = kScanCols / 8;
    extern __shared__ __align__(16) unsigned char raw[];
    const int DP = dim + 8, VP = kScanCols + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(raw);          // [16][DP]
    __nv_bfloat16* Ks = Qs + kChunk * DP;                                // [16][DP]
    __nv_bfloat16* Sb = Ks + kChunk * DP;                                // [dim][VP]
    __nv_bfloat16* Vs = Sb + dim * VP;                                   // [16][VP]
    float* As = reinterpret_cast<float*>(Vs + kChunk * VP);              // [16][16]
    float* Ds = As + kChunk * kChunk;                                    // [dim]
    constexpr int W = MODE == 0 ? 3 : 4;
    const int req = per_request[W * blockIdx.z];
    if (req < 0) return;
    const int chunk0 = per_request[W * blockIdx.z + 1], nchunks = per_request[W * blockIdx.z + 2];
    const int h = blockIdx.y, col0 = blockIdx.x * kScanCols;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int first = cu[req] + (MODE == 0 ? 0 : per_request[W * blockIdx.z + 3]), last = cu[req + 1];
    // where the state comes from and goes to: the request's slot, or the segment's entry of the scratch
    float* sfrom = MODE == 0 ? state + ((size_t)slots[req] * H + h) * dim * vdim
                             : seg_state + ((size_t)blockIdx.z * H + h) * dim * vdim;
    const bool fresh = MODE == 1 || (MODE == 0 && start_pos[req] == 0);
    float* state_ = sfrom;
    const size_t sbase = 0;
    float pd[2] = {1.f, 1.f};                               // MODE 1: the product of the chunks' decays
    float S[MT][NT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int d = (warp * MT + m) * 16 + g + (e >> 1) * 8, c = col0 + nt * 8 + 2 * t + (e & 1);
                S[m][nt][e] = (!fresh && d < dim && c < vdim) ? state_[sbase + (size_t)d * vdim + c] : 0.f;
            }
    // The next chunk's operands travel from global memory to registers while this chunk is computed (16-byte pieces of
    // q e^{b} and k e^{..}, which are contiguous; v, A and the chunk's decay by plain loads).
    constexpr int kQK = 4;                                 // 16-byte pieces of a [16][dim] tile per thread: dim <= 256
    uint4 rq[kQK], rk[kQK];
    __nv_bfloat16 rv[4];
    float ra[2], rd[2];
    const int pieces = dim / 8;                            // per row
    auto fetch = [&](int ci) {
        const int t0 = first + ci * kChunk;
        const int n = min(kChunk, last - t0);
#pragma unroll
        for (int u = 0; u < kQK; ++u) {
            const int i = threadIdx.x + u * 128;
            rq[u] = rk[u] = make_uint4(0, 0, 0, 0);
            if (i < kChunk * pieces) {
                const int j = i / pieces, pc = i % pieces;
                if (j < n) {
                    const size_t at = ((size_t)(t0 + j) * H + h) * dim + pc * 8;
                    rq[u] = *reinterpret_cast<const uint4*>(q_in + at);
                    rk[u] = *reinterpret_cast<const uint4*>(k_end + at);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = threadIdx.x + u * 128, j = i / kScanCols, c = i % kScanCols;
            rv[u] = (j < n && col0 + c < vdim) ? v[(size_t)(t0 + j) * v_stride + h * vdim + col0 + c] : __float2bfloat16_rn(0.f);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int i = threadIdx.x + u * 128, r = i / kChunk;
            ra[u] = r < n ? A[((size_t)(t0 + r) * H + h) * kChunk + i % kChunk] : 0.f;
            const int d = threadIdx.x + u * 128;
            rd[u] = d < dim ? D[((size_t)(chunk0 + ci) * H + h) * dim + d] : 0.f;
        }
    };
    fetch(0);
    for (int ci = 0; ci < nchunks; ++ci) {
        const int t0 = first + ci * kChunk;
        const int n = min(kChunk, last - t0);
        __syncthreads();                                   // the chunk before is done with the shared tiles
#pragma unroll
        for (int u = 0; u < kQK; ++u) {
            const int i = threadIdx.x + u * 128;
            if (i < kChunk * pieces) {
                const int j = i / pieces, pc = i % pieces;
                *reinterpret_cast<uint4*>(Qs + j * DP + pc * 8) = rq[u];
                *reinterpret_cast<uint4*>(Ks + j * DP + pc * 8) = rk[u];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = threadIdx.x + u * 128;
            Vs[(i / kScanCols) * VP + i % kScanCols] = rv[u];
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            As[threadIdx.x + u * 128] = ra[u];
            if (threadIdx.x + u * 128 < dim) { Ds[threadIdx.x + u * 128] = rd[u]; pd[u] *= rd[u]; }
        }
        if (ci + 1 < nchunks) fetch(ci + 1);
        // the state as it stands before this chunk, rounded, as the operand of the output product
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const int r0 = (warp * MT + m) * 16 + g;
            if (MODE != 1 && r0 - g < dim) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int c = nt * 8 + 2 * t;
                    *reinterpret_cast<__nv_bfloat162*>(Sb + r0 * VP + c) = __floats2bfloat162_rn(S[m][nt][0], S[m][nt][1]);
                    *reinterpret_cast<__nv_bfloat162*>(Sb + (r0 + 8) * VP + c) = __floats2bfloat162_rn(S[m][nt][2], S[m][nt][3]);
                }
            }
        }
        __syncthreads();
        // o[16 tokens][8 columns of this warp] = Qs Sb + As Vs
        if (MODE != 1) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const int cw = warp * 8;
            for (int kk = 0; kk < dim; kk += 16) {
                uint32_t a[4];
                a[0] = *reinterpret_cast<const uint32_t*>(Qs + g * DP + kk + 2 * t);
                a[1] = *reinterpret_cast<const uint32_t*>(Qs + (g + 8) * DP + kk + 2 * t);
                a[2] = *reinterpret_cast<const uint32_t*>(Qs + g * DP + kk + 2 * t + 8);
                a[3] = *reinterpret_cast<const uint32_t*>(Qs + (g + 8) * DP + kk + 2 * t + 8);
                const uint32_t b0 = pack2(Sb[(kk + 2 * t) * VP + cw + g], Sb[(kk + 2 * t + 1) * VP + cw + g]);
                const uint32_t b1 = pack2(Sb[(kk + 2 * t + 8) * VP + cw + g], Sb[(kk + 2 * t + 9) * VP + cw + g]);
                mma_bf16_16816(acc, a, b0, b1);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = g + (e >> 1) * 8, c = cw + 2 * t + (e & 1);
                float s = acc[e];
                for (int j = 0; j <= i; ++j) s += As[i * kChunk + j] * to_f32(Vs[j * VP + c]);
                if (i < n && col0 + c < vdim) o[((size_t)(t0 + i) * H + h) * vdim + col0 + c] = s;
            }
        }
        // S <- diag(D) S + Ks^T Vs
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const int r0 = (warp * MT + m) * 16 + g;
            if (r0 - g < dim) {
                const float d0 = Ds[r0], d1 = Ds[r0 + 8];
                uint32_t a[4];
                a[0] = pack2(Ks[(2 * t) * DP + r0], Ks[(2 * t + 1) * DP + r0]);
                a[1] = pack2(Ks[(2 * t) * DP + r0 + 8], Ks[(2 * t + 1) * DP + r0 + 8]);
                a[2] = pack2(Ks[(2 * t + 8) * DP + r0], Ks[(2 * t + 9) * DP + r0]);
                a[3] = pack2(Ks[(2 * t + 8) * DP + r0 + 8], Ks[(2 * t + 9) * DP + r0 + 8]);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    S[m][nt][0] *= d0; S[m][nt][1] *= d0; S[m][nt][2] *= d1; S[m][nt][3] *= d1;
                    const uint32_t b0 = pack2(Vs[(2 * t) * VP + nt * 8 + g], Vs[(2 * t + 1) * VP + nt * 8 + g]);
                    const uint32_t b1 = pack2(Vs[(2 * t + 8) * VP + nt * 8 + g], Vs[(2 * t + 9) * VP + nt * 8 + g]);
                    mma_bf16_16816(S[m][nt], a, b0, b1);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int d = (warp * MT + m) * 16 + g + (e >> 1) * 8, c = col0 + nt * 8 + 2 * t + (e & 1);
                if (MODE != 2 && d < dim && c < vdim) state_[sbase + (size_t)d * vdim + c] = S[m][nt][e];
            }
    if (MODE == 1 && blockIdx.x == 0) {
#pragma unroll
        for (int u = 0; u < 2; ++u)
            if (threadIdx.x + u * 128 < dim) seg_decay[((size_t)blockIdx.z * H + h) * dim + threadIdx.x + u * 128] = pd[u];
    }
}

// Between the two passes over segments: start states from end states.  per_request: int32 [m, 3] (request, its first
// segment, its segments).  For every state element: s = the slot's state (0 for a request that starts at position 0);
// for each segment: swap(seg_state[segment], s) and s = seg_decay[segment] * s_before + end state; at last the slot's
// state = s.  grid (ceil(dim * vdim / 256), H, requests)
__global__ void gla_segment_pass_kernel(float* seg_state, const float* __restrict__ seg_decay, float* state,
                                        const int* __restrict__ start_pos, const int* __restrict__ slots,
                                        const int* __restrict__ per_request, int H, int dim, int vdim) {
    const int req = per_request[3 * blockIdx.z];
    if (req < 0) return;
    const int seg0 = per_request[3 * blockIdx.z + 1], nseg = per_request[3 * blockIdx.z + 2];
    const int h = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dim * vdim) return;
    const int d = i / vdim;
    float* slot = state + ((size_t)slots[req] * H + h) * dim * vdim + i;
    float s = start_pos[req] == 0 ? 0.f : *slot;
    for (int g = seg0; g < seg0 + nseg; ++g) {
        float* e = seg_state + ((size_t)g * H + h) * dim * vdim + i;
        const float end = *e;
        *e = s;
        s = seg_decay[((size_t)g * H + h) * dim + d] * s + end;
    }
    *slot = s;
}

// Chunked form over the long portions of a step (bfloat16).  q, k, v: column views of one projection buffer; z as for
// the scan; chunks: int32 [num_chunks, 2] (request, first token within its portion; request -1: nothing);
// per_request: int32 [num_long, 3] (request, its first chunk, its number of chunks).  Scratch: q_in, k_end
// [tokens, H, dim] bfloat16, A float32 [tokens, H, 16], D float32 [num_chunks, H, dim].  dim: a multiple of 16, <= 256.
extern "C" int lb_gla_chunked(const void* q, const void* k, const void* v, long row_stride, const float* z, float* o, float* state,
                              const int* cu, const int* start_pos, const int* slots, const int* chunks, int num_chunks,
                              const int* per_request, int num_long, void* q_in, void* k_end, float* A, float* D, int H, int dim,
                              int vdim, float tau, float q_scale, const int* segments, int num_segments, float* seg_state,
                              float* seg_decay, const float* head_decay, void* stream) {
    if (num_chunks <= 0 || num_long <= 0) return kOk;
    if (H <= 0 || dim <= 0 || vdim <= 0 || !(tau > 0.f) || dim % 16) return kBadSize;
    if (dim > 256) return kTooLarge;
    cudaStream_t st = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
    {
        const size_t smem = (size_t)3 * kChunk * dim * sizeof(float);
        static size_t have = 0;
        ensure_dynamic_smem(gla_chunk_prepare_kernel, smem, have);
        gla_chunk_prepare_kernel<<<dim3(num_chunks, H), 128, smem, st>>>((const bf*)q, (const bf*)k, row_stride, z, cu, chunks,
                                                                        (bf*)q_in, (bf*)k_end, A, D, H, dim, 1.f / tau, q_scale, head_decay);
        const int rc = launch_status();
        if (rc != 0) return rc;
    }
    const size_t smem = ((size_t)2 * kChunk * (dim + 8) + (size_t)dim * (kScanCols + 8) + (size_t)kChunk * (kScanCols + 8)) * sizeof(bf)
                        + ((size_t)kChunk * kChunk + dim) * sizeof(float);
    dim3 grid((vdim + kScanCols - 1) / kScanCols, H, num_long);
#define LB_SCAN(MT_, MODE_, LIST_) { static size_t have = 0; ensure_dynamic_smem(gla_chunk_scan_kernel<MT_, MODE_>, smem, have); \
        gla_chunk_scan_kernel<MT_, MODE_><<<grid, 128, smem, st>>>((const bf*)q_in, (const bf*)k_end, (const bf*)v, row_stride, A, D, o, \
            state, cu, start_pos, slots, LIST_, H, dim, vdim, seg_state, seg_decay); }
#define LB_SCAN_MODE(MODE_, LIST_) { if (dim <= 64) LB_SCAN(1, MODE_, LIST_) else if (dim <= 128) LB_SCAN(2, MODE_, LIST_) else LB_SCAN(4, MODE_, LIST_) }
    if (segments == nullptr || num_segments <= 0) {
        LB_SCAN_MODE(0, per_request)
        return launch_status();
    }
    // a lone long prompt: its segments side by side, twice, with the pass over their states between
    grid.z = num_segments;
    LB_SCAN_MODE(1, segments)
    int rc = launch_status();
    if (rc != 0) return rc;
    gla_segment_pass_kernel<<<dim3((dim * vdim + 255) / 256, H, num_long), 256, 0, st>>>(seg_state, seg_decay, state, start_pos, slots,
                                                                                        per_request, H, dim, vdim);
    rc = launch_status();
    if (rc != 0) return rc;
    LB_SCAN_MODE(2, segments)
#undef LB_SCAN_MODE
#undef LB_SCAN
    return launch_status();
}
