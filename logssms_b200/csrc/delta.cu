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
//  delta_prepare   : a warp per (token, value head), all of them side by side: the row
//                    [q^ (DP) | k^ (DP) | g (DP) | b | <k^, q^> | 0 | 0] in 32-bit, DP = 16 * DS key channels (zeros past
//                    `dim`), and the head's values in 32-bit.
//  delta_scan_rows : the same ownership as delta_scan with 4 to 16 state rows a thread (by the key channels; DS threads of
//                    a warp share a column); the prepared rows and values of the next kTok tokens arrive by cp.async
//                    in a second buffer while the current ones are used.  A thread's rows are interleaved in fours
//                    (row 4 DS j + 4 s + i, i = 0..3) so that the 128-bit shared-memory reads of the DS threads of a
//                    column are one contiguous run.
#include "lb200/common.cuh"
using namespace lb200;

constexpr int kDeltaTokens = 8;

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename T, typename TB, int R, int DS>
__global__ void delta_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long row_stride,
                                  const float* __restrict__ z, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                  const TB* __restrict__ beta, long beta_stride, float* __restrict__ o, float* state,
                                  const int* __restrict__ cu, const int* __restrict__ start_pos, const int* __restrict__ slots,
                                  const int* __restrict__ request_list, int H, int Hk, int dim, int vdim, float q_scale, float unit_eps, int zdim) {
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
            const int zc = zdim == 1 ? 0 : d;           // one decay per head: every key channel reads the same column
            gs[i] = d < dim ? expf(-rate * softplus_f(z[((size_t)(t0 + tt) * H + h) * zdim + zc] + dt_bias[h * zdim + zc])) : 0.f;
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
                             int dim, int vdim, float q_scale, float unit_eps, int zdim, cudaStream_t stream) {
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
                                                                     request_list, H, Hk, dim, vdim, q_scale, unit_eps, zdim);
    return launch_status();
}

// --------------------------------------------------------------------------- prompt portions
constexpr int kMinPadded = 16;                       // key channels are padded to a power of two, this at least

__device__ __forceinline__ unsigned delta_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void delta_cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(delta_smem_u32(dst)), "l"(src));
}
__device__ __forceinline__ void delta_cp4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(delta_smem_u32(dst)), "l"(src));
}
__device__ __forceinline__ void delta_cp_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void delta_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

// A warp per (token, value head).  prepared: [tokens, H, 3 DP + 4]; values: [tokens, H * vdim].
template <typename T, typename TB>
__global__ void delta_prepare_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long row_stride,
                                     const float* __restrict__ z, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                     const TB* __restrict__ beta, long beta_stride, float* __restrict__ prepared, float* __restrict__ values,
                                     long pairs, int H, int Hk, int dim, int vdim, int DP, float q_scale, float unit_eps, int zdim) {
    const int lane = threadIdx.x & 31;
    const long pair = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= pairs) return;
    const long t = pair / H;
    const int h = (int)(pair % H), hk = h / (H / Hk);
    const T* qr = q + t * row_stride + (size_t)hk * dim;
    const T* kr = k + t * row_stride + (size_t)hk * dim;
    float qq = 0.f, kk = 0.f, qk = 0.f;
    for (int d = lane; d < dim; d += 32) {
        const float a = to_f32(qr[d]), e = to_f32(kr[d]);
        qq += a * a; kk += e * e; qk += a * e;
    }
    qq = warp_sum(qq); kk = warp_sum(kk); qk = warp_sum(qk);
    const float qn = q_scale / sqrtf(qq + unit_eps), kn = 1.f / sqrtf(kk + unit_eps), rate = expf(A_log[h]);
    float* row = prepared + (size_t)pair * (3 * DP + 4);
    const float* zr = z + ((size_t)t * H + h) * zdim;
    for (int d = lane; d < DP; d += 32) {
        const bool in = d < dim;
        row[d] = in ? to_f32(qr[d]) * qn : 0.f;
        row[DP + d] = in ? to_f32(kr[d]) * kn : 0.f;
        const int zc = zdim == 1 ? 0 : d;
        row[2 * DP + d] = in ? expf(-rate * softplus_f(zr[zc] + dt_bias[h * zdim + zc])) : 0.f;
    }
    if (lane < 4) {
        float x = 0.f;
        if (lane == 0) x = 1.f / (1.f + expf(-to_f32(beta[t * beta_stride + h])));
        if (lane == 1) x = qk * qn * kn;
        row[3 * DP + lane] = x;
    }
    const T* vr = v + t * row_stride + (size_t)h * vdim;
    float* orow = values + ((size_t)t * H + h) * vdim;
    for (int c = lane; c < vdim; c += 32) orow[c] = to_f32(vr[c]);
}

// A CTA owns (request, head, blockDim.x / DS value columns).
template <int R, int DS, int TOK>
__global__ void __launch_bounds__(128) delta_scan_rows_kernel(const float* __restrict__ prepared, const float* __restrict__ values,
                                                              float* __restrict__ o, float* state,
                                                              const int* __restrict__ cu, const int* __restrict__ start_pos,
                                                              const int* __restrict__ slots, const int* __restrict__ request_list,
                                                              int H, int dim, int vdim) {
    constexpr int DP = R * DS, ROW = 3 * DP + 4, PIECES = ROW / 4, Q = R / 4;
    extern __shared__ __align__(16) float sm[];
    const int cols = blockDim.x / DS;
    float* rows = sm;                                // [2][TOK][ROW]
    float* vals = sm + 2 * TOK * ROW;                // [2][TOK][cols]
    const int b = request_list ? request_list[blockIdx.z] : blockIdx.z;
    if (b < 0) return;
    const int h = blockIdx.y;
    const int col_local = threadIdx.x / DS, s = threadIdx.x % DS;
    const int c = blockIdx.x * cols + col_local;
    const int first = cu[b], last = cu[b + 1];
    if (first >= last) return;
    const size_t sbase = ((size_t)slots[b] * H + h) * dim * vdim;
    const bool fresh = start_pos[b] == 0;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = (r >> 2) * 4 * DS + 4 * s + (r & 3);
        S[r] = (!fresh && d < dim && c < vdim) ? state[sbase + (size_t)d * vdim + c] : 0.f;
    }
    auto fetch = [&](int t0, int buf) {
        const int n = min(TOK, last - t0);
        float* dst = rows + buf * TOK * ROW;
        for (int i = threadIdx.x; i < n * PIECES; i += blockDim.x) {
            const int tt = i / PIECES, piece = i % PIECES;
            delta_cp16(dst + tt * ROW + piece * 4, prepared + ((size_t)(t0 + tt) * H + h) * ROW + piece * 4);
        }
        float* vd = vals + buf * TOK * cols;
        for (int i = threadIdx.x; i < n * cols; i += blockDim.x) {
            const int tt = i / cols, cc = blockIdx.x * cols + i % cols;
            if (cc < vdim) delta_cp4(vd + i, values + ((size_t)(t0 + tt) * H + h) * vdim + cc);
        }
        delta_cp_commit();
    };
    fetch(first, 0);
    int buf = 0;
    for (int t0 = first; t0 < last; t0 += TOK, buf ^= 1) {
        if (t0 + TOK < last) { fetch(t0 + TOK, buf ^ 1); delta_cp_wait<1>(); } else { delta_cp_wait<0>(); }
        __syncthreads();
        const int n = min(TOK, last - t0);
        const float* base = rows + buf * TOK * ROW;
        const float* vd = vals + buf * TOK * cols + col_local;
        for (int tt = 0; tt < n; ++tt) {
            const float4* qr = reinterpret_cast<const float4*>(base + tt * ROW) + s;
            const float4* kr = qr + DP / 4;
            const float4* gr = kr + DP / 4;
            float4 kv[Q];
            float a[Q], e[Q];
#pragma unroll
            for (int j = 0; j < Q; ++j) {
                const float4 g = gr[j * DS], q4 = qr[j * DS];
                kv[j] = kr[j * DS];
                S[4 * j] *= g.x; S[4 * j + 1] *= g.y; S[4 * j + 2] *= g.z; S[4 * j + 3] *= g.w;
                a[j] = kv[j].x * S[4 * j] + kv[j].y * S[4 * j + 1] + kv[j].z * S[4 * j + 2] + kv[j].w * S[4 * j + 3];
                e[j] = q4.x * S[4 * j] + q4.y * S[4 * j + 1] + q4.z * S[4 * j + 2] + q4.w * S[4 * j + 3];
            }
            float dot_k, dot_q;
            if constexpr (Q == 4) { dot_k = (a[0] + a[1]) + (a[2] + a[3]); dot_q = (e[0] + e[1]) + (e[2] + e[3]); }
            else if constexpr (Q == 2) { dot_k = a[0] + a[1]; dot_q = e[0] + e[1]; }
            else { dot_k = a[0]; dot_q = e[0]; }
#pragma unroll
            for (int off = 1; off < DS; off <<= 1) {
                dot_k += __shfl_xor_sync(0xffffffffu, dot_k, off);
                dot_q += __shfl_xor_sync(0xffffffffu, dot_q, off);
            }
            const float2 gate = *reinterpret_cast<const float2*>(base + tt * ROW + 3 * DP);      // b, <k^, q^>
            const float u = gate.x * (vd[tt * cols] - dot_k);
#pragma unroll
            for (int j = 0; j < Q; ++j) {
                S[4 * j] += kv[j].x * u; S[4 * j + 1] += kv[j].y * u; S[4 * j + 2] += kv[j].z * u; S[4 * j + 3] += kv[j].w * u;
            }
            if (s == 0 && c < vdim) o[((size_t)(t0 + tt) * H + h) * vdim + c] = dot_q + u * gate.y;
        }
        __syncthreads();                             // the buffer is fetched into again in the next round
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = (r >> 2) * 4 * DS + 4 * s + (r & 3);
        if (d < dim && c < vdim) state[sbase + (size_t)d * vdim + c] = S[r];
    }
}

template <int R, int DS, int TOK>
static int launch_delta_scan_rows(const float* prepared, const float* values, float* o, float* state, const int* cu, const int* start_pos, const int* slots,
                                  const int* request_list, int num_requests, int H, int dim, int vdim, cudaStream_t stream) {
    const int threads = min(128, (vdim * DS + 31) / 32 * 32);
    const int cols = threads / DS;
    dim3 grid((vdim + cols - 1) / cols, H, num_requests);
    const size_t smem = (size_t)2 * TOK * (3 * R * DS + 4 + cols) * sizeof(float);
    static size_t have = 0;
    ensure_dynamic_smem(delta_scan_rows_kernel<R, DS, TOK>, smem, have);
    delta_scan_rows_kernel<R, DS, TOK><<<grid, threads, smem, stream>>>(prepared, values, o, state, cu, start_pos, slots, request_list, H, dim, vdim);
    return launch_status();
}

// The long portions of a step: the requests of `request_list` (all, if null).  Operands as in lb_delta_scan, plus
// prepared: float32 [tokens, H, 3 DP + 4] (DP: the power of two that reaches dim, 16 at least) and values: float32
// [tokens, H*vdim], both scratch.  Every token of the step is prepared, the listed requests are scanned.  `rows`: state
// rows a thread owns (4, 8 or 16; 0: chosen here).
extern "C" int lb_delta_scan_rows(const void* q, const void* k, const void* v, long row_stride, const float* z, const float* dt_bias,
                                  const float* A_log, const void* beta, long beta_stride, int beta_f32, float* prepared, float* values, float* o,
                                  float* state, const int* cu, const int* start_pos, const int* slots, const int* request_list,
                                  int num_requests, long tokens, int H, int Hk, int dim, int vdim, float q_scale, float unit_eps,
                                  int rows, int zdim, int dtype, void* stream) {
    if (num_requests <= 0 || tokens <= 0) return kOk;
    if (H <= 0 || Hk <= 0 || H % Hk || dim <= 0 || vdim <= 0 || H > 65535 || num_requests > 65535 || (zdim != dim && zdim != 1)) return kBadSize;
    if (dim > 512) return kTooLarge;
    cudaStream_t st = (cudaStream_t)stream;
    int DP = kMinPadded;
    while (DP < dim) DP <<= 1;
    if (rows == 0) rows = DP <= 64 ? 4 : (DP == 256 ? 8 : 16);     // measured: the fewer rows, the fewer instructions on the chain;
                                                                   // past 64 channels the longer reduction over DS lanes outweighs it
    if ((rows != 4 && rows != 8 && rows != 16) || DP / rows > 32) return kBadSize;
    const long pairs = tokens * H;
    const int warps = 4;
    const unsigned blocks = (unsigned)((pairs + warps - 1) / warps);
#define LB_PREPARE(TB_) delta_prepare_kernel<T, TB_><<<blocks, warps * 32, 0, st>>>((const T*)q, (const T*)k, (const T*)v, row_stride, z, \
        dt_bias, A_log, (const TB_*)beta, beta_stride, prepared, values, pairs, H, Hk, dim, vdim, DP, q_scale, unit_eps, zdim)
    LB_DISPATCH_DTYPE(dtype, { if (beta_f32) LB_PREPARE(float); else LB_PREPARE(T); });
#undef LB_PREPARE
    const int status = launch_status();
    if (status != kOk) return status;
#define LB_ROWS(R_, DS_, TOK_) case (R_) * 64 + (DS_): return launch_delta_scan_rows<R_, DS_, TOK_>(prepared, values, o, state, cu, start_pos, slots, \
        request_list, num_requests, H, dim, vdim, st)
    switch (rows * 64 + DP / rows) {
        LB_ROWS(4, 4, 16); LB_ROWS(4, 8, 16); LB_ROWS(4, 16, 16); LB_ROWS(4, 32, 16);
        LB_ROWS(8, 2, 16); LB_ROWS(8, 4, 16); LB_ROWS(8, 8, 16); LB_ROWS(8, 16, 16); LB_ROWS(8, 32, 8);
        LB_ROWS(16, 1, 16); LB_ROWS(16, 2, 16); LB_ROWS(16, 4, 16); LB_ROWS(16, 8, 16); LB_ROWS(16, 16, 8); LB_ROWS(16, 32, 8);
        default: return kBadSize;
    }
#undef LB_ROWS
}

// --------------------------------------------------------------------------- prompt portions in chunks of 8 tokens
// With L_t[d] the running sum of the log-decays inside a chunk (inclusive) and S0 the state the chunk starts from,
//     S'_t = diag(e^{L_t}) S0 + sum_{s<t} diag(e^{L_t - L_s}) k^_s u_s^T            (the state the write of token t meets)
//     u_t  = b_t (v_t - (k^_t e^{L_t})^T S0) - sum_{s<t} A_ts u_s,     A_ts = b_t sum_d k^_t[d] k^_s[d] e^{L_t[d] - L_s[d]}
//     o_t  = (q^_t e^{L_t})^T S0 + sum_{s<=t} B_ts u_s,                B_ts = sum_d q^_t[d] k^_s[d] e^{L_t[d] - L_s[d]}
//     S_end = diag(e^{L_end}) S0 + sum_s (k^_s e^{L_end - L_s}) u_s^T
// and every exponent is <= 0 whatever the decays are.  All of it is 32-bit; the sums are those of the token-by-token
// form in another order.  What this buys: the two dot products over the key channels of ALL tokens of a chunk are
// reduced across a column's threads in one round (their partial sums are independent), where the token-by-token form
// has one dependent round per token.  Time follows the instructions a warp issues per token (one warp per scheduler,
// an instruction every four cycles or so), so nothing is computed twice: the chunk's 16 sums are reduced by halving,
// after which each of 16 lanes holds one whole sum, and u follows by forward substitution ACROSS those lanes (token j's
// u is handed to all of them by one shuffle, each lane adds its own coefficient times it).
//  delta_chunk_prepare : one CTA per (chunk, head), all chunks of a step side by side: the record
//                        [q^ e^L (C x DP) | k^ e^L (C x DP) | k^ e^{L_end - L} (C x DP) | e^{L_end} (DP) | -A (C x C) | B (C x C) | b (C)]
//                        and the head's values in 32-bit.  Tokens past the portion's end are rows of zeros with b = 0
//                        and no decay: they change nothing.
//  delta_chunk_scan    : a CTA owns (request, head, 128 / DS value columns) and walks the request's chunks in order; a
//                        thread owns R = 4 or 8 state rows of one column, DS = 16 or 32 threads of a warp share a column
//                        (DP = R DS >= 64 key channels, zeros past `dim`).  The next chunk's record arrives by cp.async
//                        in a second buffer while this one is used.
constexpr int kDeltaChunk = 8;

template <typename T, typename TB>
__global__ void __launch_bounds__(128) delta_chunk_prepare_kernel(
        const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long row_stride, const float* __restrict__ z,
        const float* __restrict__ dt_bias, const float* __restrict__ A_log, const TB* __restrict__ beta, long beta_stride,
        const int* __restrict__ cu, const int* __restrict__ chunks, float* __restrict__ records, float* __restrict__ values,
        int H, int Hk, int dim, int vdim, int DP, float q_scale, float unit_eps, int zdim) {
    constexpr int C = kDeltaChunk;
    extern __shared__ float sm[];
    float* L = sm;                                   // [C][DP] log-decays, then their running sums
    float* qs = L + C * DP;                          // [C][DP] unit queries (scaled)
    float* ks = qs + C * DP;                         // [C][DP] unit keys
    float* bs = ks + C * DP;                         // [C]
    const int c = blockIdx.x, h = blockIdx.y, hk = h / (H / Hk);
    const int req = chunks[2 * c];
    if (req < 0) return;
    const int t0 = cu[req] + chunks[2 * c + 1];
    const int n = min(C, cu[req + 1] - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int j = warp; j < C; j += nwarps) {
        float qn = 0.f, kn = 0.f;
        const T* qr = q + (size_t)(t0 + j) * row_stride + (size_t)hk * dim;
        const T* kr = k + (size_t)(t0 + j) * row_stride + (size_t)hk * dim;
        if (j < n) {
            float qq = 0.f, kk = 0.f;
            for (int d = lane; d < dim; d += 32) {
                const float a = to_f32(qr[d]), e = to_f32(kr[d]);
                qq += a * a; kk += e * e;
            }
            qq = warp_sum(qq); kk = warp_sum(kk);
            qn = q_scale / sqrtf(qq + unit_eps); kn = 1.f / sqrtf(kk + unit_eps);
        }
        for (int d = lane; d < DP; d += 32) {
            const bool in = j < n && d < dim;
            qs[j * DP + d] = in ? to_f32(qr[d]) * qn : 0.f;
            ks[j * DP + d] = in ? to_f32(kr[d]) * kn : 0.f;
        }
        if (lane == 0) bs[j] = j < n ? 1.f / (1.f + expf(-to_f32(beta[(size_t)(t0 + j) * beta_stride + h]))) : 0.f;
    }
    const float rate = expf(A_log[h]);
    for (int i = threadIdx.x; i < C * DP; i += blockDim.x) {
        const int j = i / DP, d = i % DP;
        const int zc = zdim == 1 ? 0 : d;
        L[i] = (j < n && d < dim) ? -rate * softplus_f(z[((size_t)(t0 + j) * H + h) * zdim + zc] + dt_bias[h * zdim + zc]) : 0.f;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < DP; d += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < C; ++j) { acc += L[j * DP + d]; L[j * DP + d] = acc; }
    }
    __syncthreads();
    const int REC = 3 * C * DP + DP + 2 * C * C + C;
    float* rec = records + ((size_t)c * H + h) * REC;
    for (int i = threadIdx.x; i < C * DP; i += blockDim.x) {
        const int d = i % DP;
        const float e = expf(L[i]);
        rec[i] = qs[i] * e;
        rec[C * DP + i] = ks[i] * e;
        rec[2 * C * DP + i] = ks[i] * expf(L[(C - 1) * DP + d] - L[i]);
    }
    for (int d = threadIdx.x; d < DP; d += blockDim.x) rec[3 * C * DP + d] = expf(L[(C - 1) * DP + d]);
    float* Ao = rec + 3 * C * DP + DP;
    float* Bo = Ao + C * C;
    // a warp per pair (i, j), its lanes over the key channels
    for (int p = warp; p < C * C; p += nwarps) {
        const int i = p / C, j = p % C;
        float a = 0.f, b = 0.f;
        if (j <= i) {
            for (int d = lane; d < DP; d += 32) {
                const float w = ks[j * DP + d] * expf(L[i * DP + d] - L[j * DP + d]);
                a += ks[i * DP + d] * w;
                b += qs[i * DP + d] * w;
            }
            a = warp_sum(a); b = warp_sum(b);
        }
        if (lane == 0) { Ao[p] = j < i ? -bs[i] * a : 0.f; Bo[p] = j <= i ? b : 0.f; }
    }
    if (threadIdx.x < C) Bo[C * C + threadIdx.x] = bs[threadIdx.x];
    for (int i = threadIdx.x; i < n * vdim; i += blockDim.x) {
        const int j = i / vdim, cc = i % vdim;
        values[((size_t)(t0 + j) * H + h) * vdim + cc] = to_f32(v[(size_t)(t0 + j) * row_stride + (size_t)h * vdim + cc]);
    }
}

// grid (ceil(vdim / (128 / DS)), H, requests with long portions); per_request: (request, its first chunk, its chunks)
template <int R, int DS>
__global__ void __launch_bounds__(128) delta_chunk_scan_kernel(const float* __restrict__ records, const float* __restrict__ values,
                                                               float* __restrict__ o, float* state, const int* __restrict__ cu,
                                                               const int* __restrict__ start_pos, const int* __restrict__ slots,
                                                               const int* __restrict__ per_request, int H, int dim, int vdim) {
    constexpr int C = kDeltaChunk, DP = R * DS, Q = R / 4, REC = 3 * C * DP + DP + 2 * C * C + C, PIECES = REC / 4, cols = 128 / DS;
    extern __shared__ __align__(16) float sm[];
    float* recs = sm;                                // [2][REC]
    float* vals = sm + 2 * REC;                      // [2][C][cols]
    const int req = per_request[3 * blockIdx.z];
    if (req < 0) return;
    const int chunk0 = per_request[3 * blockIdx.z + 1], nchunks = per_request[3 * blockIdx.z + 2];
    const int h = blockIdx.y;
    const int col_local = threadIdx.x / DS, s = threadIdx.x % DS;
    const int c = blockIdx.x * cols + col_local;
    const int first = cu[req], last = cu[req + 1];
    const size_t sbase = ((size_t)slots[req] * H + h) * dim * vdim;
    const bool fresh = start_pos[req] == 0;
    float S[R];                                      // rows interleaved in fours: row 4 DS j + 4 s + i, as in delta_scan_rows
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = (r >> 2) * 4 * DS + 4 * s + (r & 3);
        S[r] = (!fresh && d < dim && c < vdim) ? state[sbase + (size_t)d * vdim + c] : 0.f;
    }
    auto fetch = [&](int ci, int buf) {
        const float* src = records + ((size_t)(chunk0 + ci) * H + h) * REC;
        float* dst = recs + buf * REC;
        for (int i = threadIdx.x; i < PIECES; i += blockDim.x) delta_cp16(dst + 4 * i, src + 4 * i);
        const int t0 = first + ci * C, n = min(C, last - t0);
        float* vd = vals + buf * C * cols;
        for (int i = threadIdx.x; i < C * cols; i += blockDim.x) {
            const int tt = i / cols, cc = blockIdx.x * cols + i % cols;
            if (tt < n && cc < vdim) delta_cp4(vd + i, values + ((size_t)(t0 + tt) * H + h) * vdim + cc);
            else vd[i] = 0.f;
        }
        delta_cp_commit();
    };
    fetch(0, 0);
    int buf = 0;
    for (int ci = 0; ci < nchunks; ++ci, buf ^= 1) {
        if (ci + 1 < nchunks) { fetch(ci + 1, buf ^ 1); delta_cp_wait<1>(); } else { delta_cp_wait<0>(); }
        __syncthreads();
        const int t0 = first + ci * C, n = min(C, last - t0);
        const float* rec = recs + buf * REC;
        const float4* Qt = reinterpret_cast<const float4*>(rec) + s;
        const float4* Kt = Qt + C * DP / 4;
        const float4* Kb = Kt + C * DP / 4;
        const float4* G4 = reinterpret_cast<const float4*>(rec + 3 * C * DP) + s;
        const float* be = rec + 3 * C * DP + DP + 2 * C * C;
        const float* vd = vals + buf * C * cols + col_local;
        float p[C], e[C], u[C];
#pragma unroll
        for (int t = 0; t < C; ++t) {
            float pp = 0.f, ee = 0.f;
#pragma unroll
            for (int j = 0; j < Q; ++j) {
                const float4 kt = Kt[t * (DP / 4) + j * DS], qt = Qt[t * (DP / 4) + j * DS];
                pp += (kt.x * S[4 * j] + kt.y * S[4 * j + 1]) + (kt.z * S[4 * j + 2] + kt.w * S[4 * j + 3]);
                ee += (qt.x * S[4 * j] + qt.y * S[4 * j + 1]) + (qt.z * S[4 * j + 2] + qt.w * S[4 * j + 3]);
            }
            p[t] = pp; e[t] = ee;
        }
        // The 16 sums (8 tokens x {<S, k^ e^L>, <S, q^ e^L>}) are reduced over the column's lanes by halving: in every stage a
        // lane keeps half of its values and hands the other half to its partner, so that lane l of 16 ends with the whole
        // sum number l (lanes 0-7: token l's key product, lanes 8-15: token l - 8's query product).
        if (DS == 32) {
#pragma unroll
            for (int t = 0; t < C; ++t) {
                p[t] += __shfl_xor_sync(0xffffffffu, p[t], 16);
                e[t] += __shfl_xor_sync(0xffffffffu, e[t], 16);
            }
        }
        const int sl = s & 15, tk = sl & 7;
        const bool reads = sl >= 8;                    // this lane ends with a read-out (else with a write's size)
        float y8[8], y4[4], y2[2], w;
#pragma unroll
        for (int i = 0; i < 8; ++i) y8[i] = (reads ? e[i] : p[i]) + __shfl_xor_sync(0xffffffffu, reads ? p[i] : e[i], 8);
        {
            const bool up = sl & 4;
#pragma unroll
            for (int i = 0; i < 4; ++i) y4[i] = (up ? y8[i + 4] : y8[i]) + __shfl_xor_sync(0xffffffffu, up ? y8[i] : y8[i + 4], 4);
        }
        {
            const bool up = sl & 2;
#pragma unroll
            for (int i = 0; i < 2; ++i) y2[i] = (up ? y4[i + 2] : y4[i]) + __shfl_xor_sync(0xffffffffu, up ? y4[i] : y4[i + 2], 2);
        }
        {
            const bool up = sl & 1;
            w = (up ? y2[1] : y2[0]) + __shfl_xor_sync(0xffffffffu, up ? y2[0] : y2[1], 1);
        }
        // Forward substitution across the lanes: lane t < 8 starts from b_t (v_t - <S0, k^_t e^L>) and lane 8 + t from token t's
        // read-out of S0; token j's finished u is handed to everyone (all lanes need it for the state), and every lane adds
        // its own coefficient times it: -A[t][j] (zero from the diagonal on) or B[t][j] (zero past the diagonal).
        if (!reads) w = be[tk] * (vd[tk * cols] - w);
        float row[C];
        {
            const float4* rp = reinterpret_cast<const float4*>(rec + 3 * C * DP + DP + (reads ? C * C : 0) + tk * C);
            const float4 r0 = rp[0], r1 = rp[1];
            row[0] = r0.x; row[1] = r0.y; row[2] = r0.z; row[3] = r0.w; row[4] = r1.x; row[5] = r1.y; row[6] = r1.z; row[7] = r1.w;
        }
        const int base = (threadIdx.x & 31) & ~(DS - 1);
#pragma unroll
        for (int j = 0; j < C; ++j) {
            u[j] = __shfl_sync(0xffffffffu, w, base | j);
            w = fmaf(row[j], u[j], w);
        }
        if (reads && s < 16 && c < vdim && tk < n) o[((size_t)(t0 + tk) * H + h) * vdim + c] = w;
#pragma unroll
        for (int j = 0; j < Q; ++j) {
            const float4 g = G4[j * DS];
            S[4 * j] *= g.x; S[4 * j + 1] *= g.y; S[4 * j + 2] *= g.z; S[4 * j + 3] *= g.w;
#pragma unroll
            for (int t = 0; t < C; ++t) {
                const float4 kb = Kb[t * (DP / 4) + j * DS];
                S[4 * j] += kb.x * u[t]; S[4 * j + 1] += kb.y * u[t]; S[4 * j + 2] += kb.z * u[t]; S[4 * j + 3] += kb.w * u[t];
            }
        }
        __syncthreads();                             // the buffer is fetched into again in the next round
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = (r >> 2) * 4 * DS + 4 * s + (r & 3);
        if (d < dim && c < vdim) state[sbase + (size_t)d * vdim + c] = S[r];
    }
}

template <int R, int DS>
static int launch_delta_chunk_scan(const float* records, const float* values, float* o, float* state, const int* cu, const int* start_pos,
                                   const int* slots, const int* per_request, int num_long, int H, int dim, int vdim, cudaStream_t stream) {
    constexpr int C = kDeltaChunk, DP = R * DS, REC = 3 * C * DP + DP + 2 * C * C + C, cols = 128 / DS;
    dim3 grid((vdim + cols - 1) / cols, H, num_long);
    const size_t smem = (size_t)2 * (REC + C * cols) * sizeof(float);
    static size_t have = 0;
    ensure_dynamic_smem(delta_chunk_scan_kernel<R, DS>, smem, have);
    delta_chunk_scan_kernel<R, DS><<<grid, 128, smem, stream>>>(records, values, o, state, cu, start_pos, slots, per_request, H, dim, vdim);
    return launch_status();
}

// The long portions of a step in chunks of 8 tokens (up to 256 key channels).  Operands as in lb_delta_scan, plus the work
// lists chunks: int32 [num_chunks, 2] (request, first token of the chunk within its portion; request -1: skipped) and
// per_request: int32 [num_long, 3] (request, its first chunk, its chunks; -1: skipped); records: float32 [num_chunks, H,
// 24 DP + DP + 136] (DP: the power of two that reaches dim, 64 at least) and values: float32 [tokens, H*vdim], both scratch.
// `rows`: state rows a thread owns (4 or 8; 0: chosen here).
extern "C" int lb_delta_scan_chunks(const void* q, const void* k, const void* v, long row_stride, const float* z, const float* dt_bias,
                                    const float* A_log, const void* beta, long beta_stride, int beta_f32, float* records, float* values,
                                    float* o, float* state, const int* cu, const int* start_pos, const int* slots, const int* chunks,
                                    int num_chunks, const int* per_request, int num_long, int H, int Hk, int dim, int vdim, float q_scale,
                                    float unit_eps, int rows, int zdim, int dtype, void* stream) {
    if (num_chunks <= 0 || num_long <= 0) return kOk;
    if (H <= 0 || Hk <= 0 || H % Hk || dim <= 0 || vdim <= 0 || H > 65535 || num_long > 65535 || (zdim != dim && zdim != 1)) return kBadSize;
    if (dim > 256) return kTooLarge;
    cudaStream_t st = (cudaStream_t)stream;
    int DP = 64;                                     // a column is shared by 16 or 32 lanes of 4 or 8 rows each
    while (DP < dim) DP <<= 1;
    const size_t smem = (size_t)(3 * kDeltaChunk * DP + kDeltaChunk) * sizeof(float);
    dim3 grid(num_chunks, H);
#define LB_PREPARE(TB_) delta_chunk_prepare_kernel<T, TB_><<<grid, 128, smem, st>>>((const T*)q, (const T*)k, (const T*)v, row_stride, z, \
        dt_bias, A_log, (const TB_*)beta, beta_stride, cu, chunks, records, values, H, Hk, dim, vdim, DP, q_scale, unit_eps, zdim)
    LB_DISPATCH_DTYPE(dtype, { if (beta_f32) LB_PREPARE(float); else LB_PREPARE(T); });
#undef LB_PREPARE
    const int status = launch_status();
    if (status != kOk) return status;
    if (rows == 0) rows = DP <= 64 ? 4 : 8;           // measured at 128 channels: 8 rows on 16 lanes beat 4 rows on 32
    if ((rows != 4 && rows != 8) || (DP / rows != 16 && DP / rows != 32)) return kBadSize;
#define LB_CHUNKS(R_, DS_) case (R_) * 64 + (DS_): return launch_delta_chunk_scan<R_, DS_>(records, values, o, state, cu, start_pos, slots, \
        per_request, num_long, H, dim, vdim, st)
    switch (rows * 64 + DP / rows) {
        LB_CHUNKS(4, 16); LB_CHUNKS(4, 32); LB_CHUNKS(8, 16); LB_CHUNKS(8, 32);
        default: return kBadSize;
    }
#undef LB_CHUNKS
}

// q, k: [tokens, Hk*dim] and v: [tokens, H*vdim], column views of one buffer (common row stride, in elements);
// z: float32 [tokens, H*zdim]; dt_bias: float32 [H*zdim] with zdim = dim (a decay per key channel) or 1 (one per head); A_log: float32 [H]; beta: [tokens, >= H] logits of the write's
// gate (float32 with `beta_f32`, else the activation dtype; row stride in elements); o: float32 [tokens, H*vdim];
// state: float32 [slots, H, dim, vdim].
extern "C" int lb_delta_scan(const void* q, const void* k, const void* v, long row_stride, const float* z, const float* dt_bias,
                             const float* A_log, const void* beta, long beta_stride, int beta_f32, float* o, float* state,
                             const int* cu, const int* start_pos, const int* slots, const int* request_list, int num_requests,
                             int H, int Hk, int dim, int vdim, float q_scale, float unit_eps, int zdim, int dtype, void* stream) {
    if (num_requests <= 0) return kOk;
    if (H <= 0 || Hk <= 0 || H % Hk || dim <= 0 || vdim <= 0 || H > 65535 || (zdim != dim && zdim != 1)) return kBadSize;
    if (dim > 512) return kTooLarge;
    cudaStream_t st = (cudaStream_t)stream;
#define LB_DELTA_B(TB_, R_, DS_) return (launch_delta_scan<T, TB_, R_, DS_>(q, k, v, row_stride, z, dt_bias, A_log, beta, beta_stride, o, \
        state, cu, start_pos, slots, request_list, num_requests, H, Hk, dim, vdim, q_scale, unit_eps, zdim, st))
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
