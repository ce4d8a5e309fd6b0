// Gated delta rule with a decay per key channel, token by token.
//
//   q^_t = q_t / sqrt(|q_t|^2 + unit_eps) * q_scale,   k^_t = k_t / sqrt(|k_t|^2 + unit_eps)      (per head, 32-bit)
//   g_t[d] = exp(-exp(A_h) * softplus(z_t[d] + dt[d]))                                             (32-bit)
//   b_t    = sigmoid(beta_t)                                                                       (32-bit, per head)
//   S      <- diag(g_t) S                             (S: [key channels, value channels] per head, 32-bit)
//   u      = b_t (v_t - S^T k^_t)
//   S      <- S + k^_t u^T
//   o_t    = S^T q^_t                                 (reads the state AFTER the token's write)
//
// Every value column of S is a recurrence of its own: u[c] and o[c] need column c only.  With S' = diag(g) S
//   u[c] = b (v[c] - <S'[:, c], k^>),   o[c] = <S'[:, c], q^> + u[c] <k^, q^>
// so a token costs one pass over the column (decay, two dot products), one reduction, and one pass to add k^ u[c].
//
//  delta_scan : the recurrence over every request's tokens of a step, state read from and written back to the
//               request's slot (a request that starts at position 0 starts from zeros whatever the slot holds).
//               A CTA owns (request, head, a tile of value columns); a thread owns R state rows of one column, DS
//               threads of a warp share a column.  The unit vectors, decays, gates and <k^, q^> of kDeltaTokens tokens
//               at a time are made in shared memory by the CTA's warps (a warp per token), so the inner loop touches
//               registers and shared memory only.  Query/key head of value head h: h / (H / Hk).  This is the kernel of
//               steps whose requests bring a token or two each (decoding).
//
// Prompt portions: the recurrence is a chain of dependent steps per value column (decay, <S'[:, c], k^>, its reduction
// over the column's threads, the gated difference, the rank-one write), about a hundred cycles a token however wide the
// GPU is, so everything that is NOT on that chain leaves the loop:
//  delta_prepare      : a CTA per token, all tokens side by side: q^ and k^ (32-bit, zero-padded to DP = 16 * DS key
//                       channels), and per value head a row [g[0..DP) | b | <k^, q^> | 0 | 0].
//  delta_scan_rows    : the same ownership as delta_scan with 16 state rows a thread; the prepared rows of the next
//                       kDeltaTokens-or-so tokens arrive by cp.async in a second buffer while the current ones are used.
//                       A thread's rows are interleaved in fours (row (r / 4) * 4 DS + 4 s + r % 4) so that the 128-bit
//                       shared-memory reads of a warp fall on distinct banks.
#include "lb200/common.cuh"
using namespace lb200;

constexpr int kDeltaTokens = 8;

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename T, typename TB, int R, int DS>
__global__ void delta_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long row_stride,
                                  const float* __restrict__ z, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                  const TB* __restrict__ beta, long beta_stride, float* __restrict__ o, float* state,
                                  const int* __restrict__ cu, const int* __restrict__ start_pos, const int* __restrict__ slots,
                                  const int* __restrict__ request_list, int H, int Hk, int dim, int vdim, float q_scale, float unit_eps) {
    constexpr int DP = R * DS;                       // key channels, padded
    extern __shared__ float sm[];
    const int cols = blockDim.x / DS;
    float* qs = sm;                                  // [kDeltaTokens][DP]
    float* ks = qs + kDeltaTokens * DP;
    float* gs = ks + kDeltaTokens * DP;
    float* vs = gs + kDeltaTokens * DP;              // [kDeltaTokens][cols]
    float* bs = vs + kDeltaTokens * cols;            // [kDeltaTokens] gate of the write
    float* kq = bs + kDeltaTokens;                   // [kDeltaTokens] <k^, q^>
    const int b = request_list ? request_list[blockIdx.z] : blockIdx.z;
    if (b < 0) return;
    const int h = blockIdx.y, hk = h / (H / Hk);
    const int col_local = threadIdx.x / DS, s = threadIdx.x % DS;
    const int c = blockIdx.x * cols + col_local;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    const int first = cu[b], last = cu[b + 1];
    const size_t sbase = ((size_t)slots[b] * H + h) * dim * vdim;
    const bool fresh = start_pos[b] == 0;
    const float rate = expf(A_log[h]);
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = s * R + r;
        S[r] = (!fresh && d < dim && c < vdim) ? state[sbase + (size_t)d * vdim + c] : 0.f;
    }
    for (int t0 = first; t0 < last; t0 += kDeltaTokens) {
        const int n = min(kDeltaTokens, last - t0);
        __syncthreads();
        // a warp per token: the two unit vectors and their product
        for (int tt = warp; tt < n; tt += nwarps) {
            const size_t row = (size_t)(t0 + tt);
            const T* qr = q + row * row_stride + (size_t)hk * dim;
            const T* kr = k + row * row_stride + (size_t)hk * dim;
            float qq = 0.f, kk = 0.f, qk = 0.f;
            for (int d = lane; d < dim; d += 32) {
                const float a = to_f32(qr[d]), e = to_f32(kr[d]);
                qq += a * a; kk += e * e; qk += a * e;
            }
            qq = warp_sum(qq); kk = warp_sum(kk); qk = warp_sum(qk);
            const float qn = q_scale / sqrtf(qq + unit_eps), kn = 1.f / sqrtf(kk + unit_eps);
            for (int d = lane; d < DP; d += 32) {
                qs[tt * DP + d] = d < dim ? to_f32(qr[d]) * qn : 0.f;
                ks[tt * DP + d] = d < dim ? to_f32(kr[d]) * kn : 0.f;
            }
            if (lane == 0) {
                kq[tt] = qk * qn * kn;
                bs[tt] = 1.f / (1.f + expf(-to_f32(beta[row * beta_stride + h])));
            }
        }
        for (int i = threadIdx.x; i < n * DP; i += blockDim.x) {
            const int tt = i / DP, d = i % DP;
            gs[i] = d < dim ? expf(-rate * softplus_f(z[((size_t)(t0 + tt) * H + h) * dim + d] + dt_bias[h * dim + d])) : 0.f;
        }
        for (int i = threadIdx.x; i < n * cols; i += blockDim.x) {
            const int tt = i / cols, cc = blockIdx.x * cols + i % cols;
            vs[i] = cc < vdim ? to_f32(v[(size_t)(t0 + tt) * row_stride + (size_t)h * vdim + cc]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float* qr = qs + tt * DP + s * R;
            const float* kr = ks + tt * DP + s * R;
            const float* gr = gs + tt * DP + s * R;
            float a = 0.f, e = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                S[r] *= gr[r];
                a += kr[r] * S[r];
                e += qr[r] * S[r];
            }
#pragma unroll
            for (int off = 1; off < DS; off <<= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, off);
                e += __shfl_xor_sync(0xffffffffu, e, off);
            }
            const float u = bs[tt] * (vs[tt * cols + col_local] - a);
#pragma unroll
            for (int r = 0; r < R; ++r) S[r] += kr[r] * u;
            if (s == 0 && c < vdim) o[((size_t)(t0 + tt) * H + h) * vdim + c] = e + u * kq[tt];
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = s * R + r;
        if (d < dim && c < vdim) state[sbase + (size_t)d * vdim + c] = S[r];
    }
}

template <typename T, typename TB, int R, int DS>
static int launch_delta_scan(const void* q, const void* k, const void* v, long row_stride, const float* z, const float* dt_bias,
                             const float* A_log, const void* beta, long beta_stride, float* o, float* state, const int* cu,
                             const int* start_pos, const int* slots, const int* request_list, int num_requests, int H, int Hk,
                             int dim, int vdim, float q_scale, float unit_eps, cudaStream_t stream) {
    // few requests: narrow tiles, so that more CTAs share the work
    const int want = (num_requests * H * ((vdim * DS + 127) / 128) < 148) ? 32 : 128;
    const int threads = min(want, (vdim * DS + 31) / 32 * 32);
    const int cols = threads / DS;
    dim3 grid((vdim + cols - 1) / cols, H, num_requests);
    const size_t smem = (size_t)kDeltaTokens * (3 * R * DS + cols + 2) * sizeof(float);
    static size_t have = 0;
    ensure_dynamic_smem(delta_scan_kernel<T, TB, R, DS>, smem, have);
    delta_scan_kernel<T, TB, R, DS><<<grid, threads, smem, stream>>>((const T*)q, (const T*)k, (const T*)v, row_stride, z, dt_bias, A_log,
                                                                     (const TB*)beta, beta_stride, o, state, cu, start_pos, slots,
                                                                     request_list, H, Hk, dim, vdim, q_scale, unit_eps);
    return launch_status();
}

// q, k: [tokens, Hk*dim] and v: [tokens, H*vdim], column views of one buffer (common row stride, in elements);
// z: float32 [tokens, H*dim]; dt_bias: float32 [H*dim]; A_log: float32 [H]; beta: [tokens, >= H] logits of the write's
// gate (float32 with `beta_f32`, else the activation dtype; row stride in elements); o: float32 [tokens, H*vdim];
// state: float32 [slots, H, dim, vdim].
extern "C" int lb_delta_scan(const void* q, const void* k, const void* v, long row_stride, const float* z, const float* dt_bias,
                             const float* A_log, const void* beta, long beta_stride, int beta_f32, float* o, float* state,
                             const int* cu, const int* start_pos, const int* slots, const int* request_list, int num_requests,
                             int H, int Hk, int dim, int vdim, float q_scale, float unit_eps, int dtype, void* stream) {
    if (num_requests <= 0) return kOk;
    if (H <= 0 || Hk <= 0 || H % Hk || dim <= 0 || vdim <= 0 || H > 65535) return kBadSize;
    if (dim > 512) return kTooLarge;
    cudaStream_t st = (cudaStream_t)stream;
#define LB_DELTA_B(TB_, R_, DS_) return (launch_delta_scan<T, TB_, R_, DS_>(q, k, v, row_stride, z, dt_bias, A_log, beta, beta_stride, o, \
        state, cu, start_pos, slots, request_list, num_requests, H, Hk, dim, vdim, q_scale, unit_eps, st))
#define LB_DELTA(R_, DS_) LB_DISPATCH_DTYPE(dtype, { if (beta_f32) LB_DELTA_B(float, R_, DS_); else LB_DELTA_B(T, R_, DS_); })
    if (dim <= 16) { LB_DELTA(16, 1); }
    else if (dim <= 32) { LB_DELTA(32, 1); }
    else if (dim <= 64) { LB_DELTA(64, 1); }
    else if (dim <= 128) { LB_DELTA(64, 2); }
    else if (dim <= 256) { LB_DELTA(64, 4); }
    else { LB_DELTA(64, 8); }
#undef LB_DELTA
#undef LB_DELTA_B
    return kOk;
}
