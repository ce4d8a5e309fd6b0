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
                                     long pairs, int H, int Hk, int dim, int vdim, int DP, float q_scale, float unit_eps) {
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
    const float* zr = z + ((size_t)t * H + h) * dim;
    for (int d = lane; d < DP; d += 32) {
        const bool in = d < dim;
        row[d] = in ? to_f32(qr[d]) * qn : 0.f;
        row[DP + d] = in ? to_f32(kr[d]) * kn : 0.f;
        row[2 * DP + d] = in ? expf(-rate * softplus_f(zr[d] + dt_bias[h * dim + d])) : 0.f;
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
                                  int rows, int dtype, void* stream) {
    if (num_requests <= 0 || tokens <= 0) return kOk;
    if (H <= 0 || Hk <= 0 || H % Hk || dim <= 0 || vdim <= 0 || H > 65535 || num_requests > 65535) return kBadSize;
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
        dt_bias, A_log, (const TB_*)beta, beta_stride, prepared, values, pairs, H, Hk, dim, vdim, DP, q_scale, unit_eps)
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
