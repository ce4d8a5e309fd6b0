// Attention over a cache of latents (one compressed row per token, shared by all heads) with a rotated key part.
//
// Per token the cache keeps c [rank] (the normalised latent) and kr [rot] (one rotated key part for all heads).
// A head's key is [W_uk,h c | kr] and its value W_uv,h c.  The kernels work in the latent space: the query's
// unrotated part is folded through W_uk,h first (qa = W_uk,h^T q, `lb_heads_matmul`), scores are
// (qa . c + q_rot . kr) * scale, the weighted sum of the c rows is expanded through W_uv,h afterwards.
//
//  latent_prepare   : per token: RMSNorm of the first `rank` columns of the down-projection -> cache "c";
//                     rotation of its last `rot` columns -> cache "kr"; rotation of every head's query part, in place
//  heads_matmul     : out[t, h, n] = sum_k a[t, h, k] * w[h, k, n]     (32-bit accumulation)
//  latent_attention : softmax attention of listed tokens over their request's pages, keys j with
//                     0 <= p - j < window (window 0: all earlier keys).  One warp per (token, head); the warps of a
//                     CTA are heads of one token and share its key tiles in shared memory; scores, softmax weights
//                     and the weighted sum are 32-bit.
#include "lb200/common.cuh"
using namespace lb200;

// grid (tokens); the rotation pairs column i with i + rd/2 among the first rd columns of a rotated part, or, with
// `neighbours`, column 2i with 2i + 1.  Without `write_cache` the row holds the queries alone (a layer that reads the
// latents another layer cached has no down-projection).
template <typename T>
__global__ void latent_prepare_kernel(T* proj, long row_stride, int q_cols, int H, int nope, int rot, int rank,
                                      const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                                      const float* __restrict__ cos_sin, int table_rows, int rd,
                                      const float* __restrict__ norm_w, float eps, T* __restrict__ c_cache,
                                      T* __restrict__ kr_cache, int write_cache, int neighbours) {
    __shared__ float red[32];
    const size_t t = blockIdx.x;
    T* row = proj + t * row_stride;
    const int pos = min(max(positions[t], 0), table_rows - 1);
    const float* cs = cos_sin + (size_t)pos * rd;
    const int half = rd >> 1;
    if (write_cache) {                                        // (uniform over the grid: no thread skips the reduction)
        const size_t slot = (size_t)slot_mapping[t];
        // latent: RMSNorm in 32-bit
        const T* d = row + q_cols;
        float ss = 0.f;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_f32(d[i]); ss += v * v; }
        ss = block_sum(ss, red);
        const float inv = 1.f / sqrtf(ss / (float)rank + eps);
        for (int i = threadIdx.x; i < rank; i += blockDim.x) c_cache[slot * rank + i] = from_f32<T>(to_f32(d[i]) * inv * norm_w[i]);
        // the shared rotated key part
        const T* kr = d + rank;
        for (int i = threadIdx.x; i < rot; i += blockDim.x) {
            float v = to_f32(kr[i]);
            if (neighbours) {
                if (i < rd) {
                    const float partner = to_f32(kr[i ^ 1]), co = cs[i >> 1], si = cs[half + (i >> 1)];
                    v = (i & 1) ? v * co + partner * si : v * co - partner * si;
                }
            } else if (i < half) v = v * cs[i] - to_f32(kr[i + half]) * cs[half + i];
            else if (i < rd) v = v * cs[i - half] + to_f32(kr[i - half]) * cs[i];
            kr_cache[slot * rot + i] = from_f32<T>(v);
        }
    }
    // every head's rotated query part, in place (a thread owns a pair)
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        const int h = i / half, j = i % half;
        T* qr = row + (size_t)h * (nope + rot) + nope;
        const int a = neighbours ? 2 * j : j, b = neighbours ? 2 * j + 1 : j + half;
        const float u = to_f32(qr[a]), w = to_f32(qr[b]);
        qr[a] = from_f32<T>(u * cs[j] - w * cs[half + j]);
        qr[b] = from_f32<T>(w * cs[j] + u * cs[half + j]);
    }
}

extern "C" int lb_latent_prepare(void* proj, long row_stride, int q_cols, int H, int nope, int rot, int rank,
                                 const int* positions, const int* slot_mapping, const float* cos_sin, int table_rows, int rd,
                                 const float* norm_w, float eps, void* c_cache, void* kr_cache, int write_cache, int neighbours,
                                 int tokens, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (H <= 0 || nope < 0 || rot < 0 || rank <= 0 || rd < 0 || rd > rot || (rd & 1)) return kBadSize;
    LB_DISPATCH_DTYPE(dtype, latent_prepare_kernel<T><<<tokens, 128, 0, (cudaStream_t)stream>>>(
        (T*)proj, row_stride, q_cols, H, nope, rot, rank, positions, slot_mapping, cos_sin, table_rows, rd, norm_w, eps,
        (T*)c_cache, (T*)kr_cache, write_cache, neighbours));
    return launch_status();
}

// grid (ceil(N / 32), H, ceil(tokens / 8)), 128 threads: 32 output columns x 4 slices of K, summed through shared
// memory (a step of few tokens then still has enough CTAs in flight to stream the weights);
// a[t*a_row + h*a_head + k]; w [H, K, N]; out[t*o_row + h*o_head + n]
constexpr int kHmTokens = 8;
template <typename T>
__global__ void __launch_bounds__(128) heads_matmul_kernel(const T* __restrict__ a, long a_row, long a_head, const T* __restrict__ w,
                                                           T* __restrict__ out, long o_row, long o_head, int tokens, int K, int N) {
    extern __shared__ float as[];                    // [kHmTokens][K], then [4][kHmTokens][32] partial sums
    float* part = as + kHmTokens * K;
    const int h = blockIdx.y, t0 = blockIdx.z * kHmTokens;
    const int nt = min(kHmTokens, tokens - t0);
    for (int i = threadIdx.x; i < kHmTokens * K; i += blockDim.x) {
        const int tt = i / K, kk = i % K;
        as[i] = tt < nt ? to_f32(a[(size_t)(t0 + tt) * a_row + (size_t)h * a_head + kk]) : 0.f;
    }
    __syncthreads();
    const int col = threadIdx.x & 31, slice = threadIdx.x >> 5;
    const int n = blockIdx.x * 32 + col;
    float acc[kHmTokens];
#pragma unroll
    for (int tt = 0; tt < kHmTokens; ++tt) acc[tt] = 0.f;
    if (n < N) {
        const T* wp = w + (size_t)h * K * N + n;
#pragma unroll 4
        for (int kk = slice; kk < K; kk += 4) {
            const float wv = to_f32(wp[(size_t)kk * N]);
#pragma unroll
            for (int tt = 0; tt < kHmTokens; ++tt) acc[tt] += as[tt * K + kk] * wv;
        }
    }
#pragma unroll
    for (int tt = 0; tt < kHmTokens; ++tt) part[(slice * kHmTokens + tt) * 32 + col] = acc[tt];
    __syncthreads();
    for (int i = threadIdx.x; i < nt * 32; i += blockDim.x) {
        const int tt = i >> 5, c = i & 31, nn = blockIdx.x * 32 + c;
        if (nn < N) {
            const float sum = (part[tt * 32 + c] + part[(kHmTokens + tt) * 32 + c])
                            + (part[(2 * kHmTokens + tt) * 32 + c] + part[(3 * kHmTokens + tt) * 32 + c]);
            out[(size_t)(t0 + tt) * o_row + (size_t)h * o_head + nn] = from_f32<T>(sum);
        }
    }
}

extern "C" int lb_heads_matmul(const void* a, long a_row, long a_head, const void* w, void* out, long o_row, long o_head,
                               int tokens, int H, int K, int N, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (H <= 0 || K <= 0 || N <= 0) return kBadSize;
    const size_t smem = ((size_t)kHmTokens * K + 4 * kHmTokens * 32) * sizeof(float);
    if (smem > 160 * 1024) return kTooLarge;
    dim3 grid((N + 31) / 32, H, (tokens + kHmTokens - 1) / kHmTokens);
    LB_DISPATCH_DTYPE(dtype, {
        static size_t have = 0;
        ensure_dynamic_smem(heads_matmul_kernel<T>, smem, have);
        heads_matmul_kernel<T><<<grid, 128, smem, (cudaStream_t)stream>>>((const T*)a, a_row, a_head, (const T*)w, (T*)out,
                                                                         o_row, o_head, tokens, K, N);
    });
    return launch_status();
}

constexpr int kLaWarps = 4;       // heads of one token per CTA
constexpr int kLaTile = 32;       // keys per tile: one per lane
constexpr int kLaMaxPieces = 16;  // rank <= 32 * 16

// grid (listed tokens, ceil(H / kLaWarps))
template <typename T>
__global__ void __launch_bounds__(kLaWarps * 32) latent_attention_kernel(
        const T* __restrict__ qa, const T* __restrict__ q_rot, long q_rot_row, long q_rot_head,
        const T* __restrict__ c_cache, const T* __restrict__ kr_cache, const int* __restrict__ block_table, int table_width,
        const int* __restrict__ token_req, const int* __restrict__ positions, const int* __restrict__ token_list,
        T* __restrict__ out, int H, int rank, int rot, int page_size, float scale, int window, const float* __restrict__ sinks) {
    extern __shared__ float sm[];
    const int D = rank + rot, DP = D + 1;
    float* qs = sm;                        // [kLaWarps][D]
    float* ks = sm + kLaWarps * D;         // [kLaTile][DP]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = token_list ? token_list[blockIdx.x] : blockIdx.x;
    if (t < 0) return;
    const int h = blockIdx.y * kLaWarps + warp;
    const bool live = h < H;
    const int p = positions[t];
    const int* pages = block_table + (size_t)token_req[t] * table_width;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    if (live) {
        for (int d = lane; d < D; d += 32)
            qs[warp * D + d] = scale * (d < rank ? to_f32(qa[((size_t)t * H + h) * rank + d])
                                                 : to_f32(q_rot[(size_t)t * q_rot_row + (size_t)h * q_rot_head + d - rank]));
    }
    const int pieces = (rank + 31) >> 5;
    float acc[kLaMaxPieces];
#pragma unroll
    for (int i = 0; i < kLaMaxPieces; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int j0 = lo; j0 <= p; j0 += kLaTile) {
        const int nvalid = min(kLaTile, p - j0 + 1);
        __syncthreads();
        for (int jj = warp; jj < nvalid; jj += kLaWarps) {
            const int j = j0 + jj;
            const size_t off = (size_t)pages[j / page_size] * page_size + j % page_size;
            for (int d = lane; d < D; d += 32)
                ks[jj * DP + d] = d < rank ? to_f32(c_cache[off * rank + d]) : to_f32(kr_cache[off * rot + d - rank]);
        }
        __syncthreads();
        if (!live) continue;
        float s = -INFINITY;
        if (lane < nvalid) {
            s = 0.f;
            const float* kr = ks + lane * DP;
            const float* qr = qs + warp * D;
            for (int d = 0; d < D; ++d) s += qr[d] * kr[d];
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);           // m = -inf at the first tile: 0
        const float pj = lane < nvalid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(pj);
#pragma unroll
        for (int i = 0; i < kLaMaxPieces; ++i) acc[i] *= corr;
        for (int jj = 0; jj < nvalid; ++jj) {
            const float pp = __shfl_sync(0xffffffffu, pj, jj);
            const float* kr = ks + jj * DP;
#pragma unroll
            for (int i = 0; i < kLaMaxPieces; ++i)
                if (i < pieces) { const int r = lane + 32 * i; if (r < rank) acc[i] += pp * kr[r]; }
        }
        m = m_new;
    }
    if (!live) return;
    if (sinks != nullptr) l += expf(sinks[h] - m);             // the sink: one more term of the denominator, no key, no value
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < kLaMaxPieces; ++i)
        if (i < pieces) { const int r = lane + 32 * i; if (r < rank) out[((size_t)t * H + h) * rank + r] = from_f32<T>(acc[i] * inv); }
}

// qa: [tokens, H, rank]; q_rot: the rotated query parts inside another buffer (row and head strides in elements);
// caches: [pages, page_size, rank] and [pages, page_size, rot]; out: [tokens, H, rank] (listed rows only)
extern "C" int lb_latent_attention(const void* qa, const void* q_rot, long q_rot_row, long q_rot_head, const void* c_cache,
                                   const void* kr_cache, const int* block_table, int table_width, const int* token_req,
                                   const int* positions, const int* token_list, int num_listed, void* out, int H, int rank,
                                   int rot, int page_size, float scale, int window, const float* sinks, int dtype, void* stream) {
    if (num_listed <= 0) return kOk;
    if (H <= 0 || rank <= 0 || rot < 0 || page_size <= 0 || window < 0) return kBadSize;
    if (rank > 32 * kLaMaxPieces) return kTooLarge;
    const int D = rank + rot;
    const size_t smem = ((size_t)kLaWarps * D + (size_t)kLaTile * (D + 1)) * sizeof(float);
    if (smem > 200 * 1024) return kTooLarge;
    dim3 grid(num_listed, (H + kLaWarps - 1) / kLaWarps);
    LB_DISPATCH_DTYPE(dtype, {
        static size_t have = 0;
        ensure_dynamic_smem(latent_attention_kernel<T>, smem, have);
        latent_attention_kernel<T><<<grid, kLaWarps * 32, smem, (cudaStream_t)stream>>>(
            (const T*)qa, (const T*)q_rot, q_rot_row, q_rot_head, (const T*)c_cache, (const T*)kr_cache, block_table,
            table_width, token_req, positions, token_list, (T*)out, H, rank, rot, page_size, scale, window, sinks);
    });
    return launch_status();
}

// ------------------------------------------------------------------------------------------------------------------
// The same attention on the tensor cores (bfloat16; rank a multiple of 32 up to 512, rot a multiple of 16).
//
// All heads of a token read the same cached rows, so the 16 rows of an `mma.sync` tile are (token, head) pairs that
// share their keys: 16 heads of one token, or 16 / H neighbouring tokens of one request with all their H heads.  A CTA
// of four warps owns one such tile and one range of its keys (`splits` ranges per tile: a decode step has few tiles).
// Per 32 keys, staged once in shared memory as [c | kr] rows: every warp computes the scores of 8 of the keys over
// the whole row length rank + rot, the row maxima meet in shared memory, the weights (32-bit, then rounded for the
// product) go to shared memory, and every warp multiplies them with its quarter of the c columns; the running output
// stays in registers.  Scores, maxima, weights and sums are 32-bit.  With one range the CTA writes the output, else
// its unnormalised part with the row's maximum and sum, which `latent_merge` puts together.
constexpr int kMmaKeys = 32;

__device__ __forceinline__ void mma_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(gmem_src) : "memory");
}
// four (two) 8x8 tiles of 16-bit values from shared memory into the fragment layout of `mma.sync`; lane 8i + r gives the
// address of row r of tile i; `_t`: every tile transposed on the way
__device__ __forceinline__ void ldsm_x4(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2_t(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ uint32_t pack_bf16(__nv_bfloat16 lo, __nv_bfloat16 hi) {
    return (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
}

// grid (token blocks, head groups, splits); NTW: 8-column output tiles per warp (rank <= 32 * NTW)
template <int NTW>
__global__ void __launch_bounds__(128) latent_attention_mma_kernel(
        const __nv_bfloat16* __restrict__ qa, long qa_row, long qa_head, const __nv_bfloat16* __restrict__ q_rot, long q_rot_row,
        long q_rot_head, const __nv_bfloat16* __restrict__ c_cache, const __nv_bfloat16* __restrict__ kr_cache,
        const int* __restrict__ block_table, int table_width, const int* __restrict__ token_req,
        const int* __restrict__ positions, const int* __restrict__ blocks, __nv_bfloat16* __restrict__ out,
        float* __restrict__ part_o, float* __restrict__ part_ml, int H, int rank, int rot, int page_size, float scale,
        int window, int splits, const float* __restrict__ sinks) {
    typedef __nv_bfloat16 bf;
    extern __shared__ __align__(16) unsigned char raw[];
    const int D = rank + rot, DP = D + 8, PP = kMmaKeys + 8;
    bf* Qs = reinterpret_cast<bf*>(raw);                    // [16][DP]
    bf* Kt0 = Qs + 16 * DP;                                 // two buffers of [32][DP]
    bf* Ps = Kt0 + 2 * kMmaKeys * DP;                       // [16][PP]
    float* red = reinterpret_cast<float*>(Ps + 16 * PP);    // [4][16]
    __shared__ int row_lo[16], row_hi[16];
    const int t0 = blocks ? blocks[2 * blockIdx.x] : blockIdx.x, ntok = blocks ? blocks[2 * blockIdx.x + 1] : 1;
    if (t0 < 0) return;
    const int nh = H >= 16 ? min(16, H - (int)blockIdx.y * 16) : H;       // heads of this tile
    const int h0 = H >= 16 ? blockIdx.y * 16 : 0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int* pages = block_table + (size_t)token_req[t0] * table_width;
    if (threadIdx.x < 16) {
        const int r = threadIdx.x, tok = r / nh;
        int lo = 1, hi = 0;                                  // an empty range: a row without a token
        if (tok < ntok) {
            hi = positions[t0 + tok];
            lo = window > 0 ? max(0, hi - window + 1) : 0;
        }
        row_lo[r] = lo; row_hi[r] = hi;
    }
    for (int i = threadIdx.x; i < 16 * D; i += blockDim.x) {
        const int r = i / D, d = i % D, tok = r / nh, h = h0 + r % nh;
        bf v = __float2bfloat16_rn(0.f);
        if (tok < ntok)
            v = d < rank ? qa[(size_t)(t0 + tok) * qa_row + (size_t)h * qa_head + d]
                         : q_rot[(size_t)(t0 + tok) * q_rot_row + (size_t)h * q_rot_head + d - rank];
        Qs[r * DP + d] = v;
    }
    const int p_hi = positions[t0 + ntok - 1], p_first = positions[t0];
    const int key_lo = window > 0 ? max(0, p_first - window + 1) : 0;
    const int tiles = (p_hi - key_lo + kMmaKeys) / kMmaKeys;
    const int per = (tiles + splits - 1) / splits;
    const int tile_lo = blockIdx.z * per, tile_hi = min(tiles, tile_lo + per);
    float acc[NTW][4];
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int ntw = rank / 32;                               // output tiles of this warp
    const int colw = warp * (rank / 4);
    __syncthreads();
    const int lo0 = row_lo[g], hi0 = row_hi[g], lo1 = row_lo[g + 8], hi1 = row_hi[g + 8];
    // key tiles come by 16-byte asynchronous copies into two buffers: the next tile travels while this one is used
    auto stage = [&](int tile, bf* dstbase) {
        const int j0 = key_lo + tile * kMmaKeys;
        // every lane looks up the cache row of one key of the tile (one trip to the page table, not one per row)
        const int jl = j0 + lane;
        const long long mine = jl <= p_hi ? (long long)pages[jl / page_size] * page_size + jl % page_size : -1;
        for (int jj = warp; jj < kMmaKeys; jj += 4) {
            const long long off = __shfl_sync(0xffffffffu, mine, jj);
            bf* dst = dstbase + jj * DP;
            if (off >= 0) {
                const bf* c4 = c_cache + off * rank;
                const bf* k4 = kr_cache + off * rot;
                for (int i = lane; i < rank / 8; i += 32) cp_async_16(dst + i * 8, c4 + i * 8);
                for (int i = lane; i < rot / 8; i += 32) cp_async_16(dst + rank + i * 8, k4 + i * 8);
            } else {
                for (int i = lane; i < D / 8; i += 32) reinterpret_cast<uint4*>(dst)[i] = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (tile_lo < tile_hi) stage(tile_lo, Kt0);
    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        const int j0 = key_lo + tile * kMmaKeys;
        bf* Kt = Kt0 + ((tile - tile_lo) & 1) * kMmaKeys * DP;
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();                                     // this tile has landed; the tile before is used up
        if (tile + 1 < tile_hi) stage(tile + 1, Kt0 + ((tile + 1 - tile_lo) & 1) * kMmaKeys * DP);
        // scores of this warp's 8 keys
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        {
            // A: the 16 query rows (tiles: rows 0-7 | 8-15 at k, then at k + 8); B: this warp's 8 keys (k, k + 8, k + 16, k + 24)
            const bf* qp = Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * DP + (lane >> 4) * 8;
            const bf* kp = Kt + (warp * 8 + (lane & 7)) * DP + (lane >> 3) * 8;
            int kk = 0;
            for (; kk + 32 <= D; kk += 32) {
                uint32_t a0[4], a1[4], b[4];
                ldsm_x4(a0, qp + kk);
                ldsm_x4(a1, qp + kk + 16);
                ldsm_x4(b, kp + kk);
                mma_16816(s, a0, b[0], b[1]);
                mma_16816(s, a1, b[2], b[3]);
            }
            if (kk < D) {
                uint32_t a0[4], b[2];
                ldsm_x4(a0, qp + kk);
                ldsm_x2(b, kp + kk);                     // (lanes 16-31 give addresses that are not used)
                mma_16816(s, a0, b[0], b[1]);
            }
        }
        const int jk = j0 + warp * 8 + 2 * t;
        s[0] = (jk >= lo0 && jk <= hi0) ? s[0] * scale : -INFINITY;
        s[1] = (jk + 1 >= lo0 && jk + 1 <= hi0) ? s[1] * scale : -INFINITY;
        s[2] = (jk >= lo1 && jk <= hi1) ? s[2] * scale : -INFINITY;
        s[3] = (jk + 1 >= lo1 && jk + 1 <= hi1) ? s[3] * scale : -INFINITY;
        float mx0 = fmaxf(s[0], s[1]), mx1 = fmaxf(s[2], s[3]);
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if (t == 0) { red[warp * 16 + g] = mx0; red[warp * 16 + g + 8] = mx1; }
        __syncthreads();
        float corr[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int r = g + 8 * e;
            const float mt = fmaxf(fmaxf(red[r], red[16 + r]), fmaxf(red[32 + r], red[48 + r]));
            const float mn = fmaxf(m[e], mt);
            corr[e] = (mn == -INFINITY) ? 1.f : expf(m[e] - mn);
            m[e] = mn;
        }
        const float p0 = m[0] == -INFINITY ? 0.f : expf(s[0] - m[0]), p1 = m[0] == -INFINITY ? 0.f : expf(s[1] - m[0]);
        const float p2 = m[1] == -INFINITY ? 0.f : expf(s[2] - m[1]), p3 = m[1] == -INFINITY ? 0.f : expf(s[3] - m[1]);
        const __nv_bfloat162 pa = __floats2bfloat162_rn(p0, p1), pb = __floats2bfloat162_rn(p2, p3);
        *reinterpret_cast<__nv_bfloat162*>(Ps + g * PP + warp * 8 + 2 * t) = pa;
        *reinterpret_cast<__nv_bfloat162*>(Ps + (g + 8) * PP + warp * 8 + 2 * t) = pb;
        // the sums take the weights as the product sees them
        l[0] = l[0] * corr[0] + __bfloat162float(pa.x) + __bfloat162float(pa.y);
        l[1] = l[1] * corr[1] + __bfloat162float(pb.x) + __bfloat162float(pb.y);
        __syncthreads();
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
            if (nt < ntw) { acc[nt][0] *= corr[0]; acc[nt][1] *= corr[0]; acc[nt][2] *= corr[1]; acc[nt][3] *= corr[1]; }
        }
#pragma unroll
        for (int ks = 0; ks < kMmaKeys; ks += 16) {
            uint32_t a[4];
            ldsm_x4(a, Ps + ((lane & 7) + ((lane >> 3) & 1) * 8) * PP + ks + (lane >> 4) * 8);
            // B: 16 keys x 8 columns per output tile, transposed on the way; two output tiles per load
            const bf* vp = Kt + (ks + (lane & 7) + ((lane >> 3) & 1) * 8) * DP + colw + (lane >> 4) * 8;
#pragma unroll
            for (int nt = 0; nt < NTW; nt += 2) {
                if (nt + 1 < ntw) {
                    uint32_t b[4];
                    ldsm_x4_t(b, vp + nt * 8);
                    mma_16816(acc[nt], a, b[0], b[1]);
                    mma_16816(acc[nt + 1], a, b[2], b[3]);
                } else if (nt < ntw) {
                    uint32_t b[2];
                    ldsm_x2_t(b, vp + nt * 8);
                    mma_16816(acc[nt], a, b[0], b[1]);
                }
            }
        }
    }
    // the rows' sums: over the four lanes that share a row, then over the warps
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        l[e] += __shfl_xor_sync(0xffffffffu, l[e], 1);
        l[e] += __shfl_xor_sync(0xffffffffu, l[e], 2);
    }
    if (t == 0) { red[warp * 16 + g] = l[0]; red[warp * 16 + g + 8] = l[1]; }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int r = g + 8 * e, tok = r / nh, h = h0 + r % nh;
        if (tok >= ntok) continue;
        float lt = red[r] + red[16 + r] + red[32 + r] + red[48 + r];
        const size_t row = (size_t)(t0 + tok) * H + h;
        if (splits == 1) {
            if (sinks != nullptr && lt > 0.f) lt += expf(sinks[h] - m[e]);       // the sink joins the denominator once
            const float inv = lt > 0.f ? 1.f / lt : 0.f;
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt)
                if (nt < ntw)
                    *reinterpret_cast<__nv_bfloat162*>(out + row * rank + colw + nt * 8 + 2 * t) =
                        __floats2bfloat162_rn(acc[nt][2 * e] * inv, acc[nt][2 * e + 1] * inv);
        } else {
            float* po = part_o + (row * splits + blockIdx.z) * rank + colw;
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt)
                if (nt < ntw) { po[nt * 8 + 2 * t] = acc[nt][2 * e]; po[nt * 8 + 2 * t + 1] = acc[nt][2 * e + 1]; }
            if (warp == 0 && t == 0) {
                part_ml[(row * splits + blockIdx.z) * 2] = m[e];
                part_ml[(row * splits + blockIdx.z) * 2 + 1] = lt;
            }
        }
    }
}

// The same for prompt portions: a CTA holds 4 / CH tiles of 16 rows (up to 64 (token, head) rows of neighbouring tokens
// of one request), so a staged key tile serves four times the rows.  A warp owns one row tile (CH = 2: two warps share
// a row tile and split the output columns): it computes all 32 scores of its rows, keeps the weights in registers (the
// accumulator layout of the score tiles is the operand layout of the next product) and its running output in
// registers; warps meet only at the one barrier per key tile that guards the two staging buffers.
// grid (token blocks, head groups); NTW: 8-column output tiles per warp (rank / CH <= 8 * NTW)
template <int NTW, int CH>
__global__ void __launch_bounds__(128) latent_attention_wide_kernel(
        const __nv_bfloat16* __restrict__ qa, long qa_row, long qa_head, const __nv_bfloat16* __restrict__ q_rot, long q_rot_row,
        long q_rot_head, const __nv_bfloat16* __restrict__ c_cache, const __nv_bfloat16* __restrict__ kr_cache,
        const int* __restrict__ block_table, int table_width, const int* __restrict__ token_req,
        const int* __restrict__ positions, const int* __restrict__ blocks, __nv_bfloat16* __restrict__ out,
        int H, int rank, int rot, int page_size, float scale, int window, const float* __restrict__ sinks) {
    typedef __nv_bfloat16 bf;
    constexpr int RT = 4 / CH, ROWS = RT * 16;
    extern __shared__ __align__(16) unsigned char raw[];
    const int D = rank + rot, DP = D + 8;
    bf* Qs = reinterpret_cast<bf*>(raw);                    // [ROWS][DP]
    bf* Kt0 = Qs + ROWS * DP;                               // two buffers of [32][DP]
    __shared__ int row_lo[ROWS], row_hi[ROWS];
    const int t0 = blocks[2 * blockIdx.x], ntok = blocks[2 * blockIdx.x + 1];
    if (t0 < 0) return;
    const int h0 = H >= 16 ? blockIdx.y * 16 : 0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int rt = warp / CH, half = warp % CH;
    const int* pages = block_table + (size_t)token_req[t0] * table_width;
    // row r of the CTA -> (token of the block, head); -1: no such row
    auto row_token = [&](int r) { const int tok = H >= 16 ? r / 16 : r / H; return (tok < ntok && (H < 16 || h0 + r % 16 < H)) ? tok : -1; };
    auto row_head = [&](int r) { return H >= 16 ? h0 + r % 16 : r % H; };
    if (threadIdx.x < ROWS) {
        const int tok = row_token(threadIdx.x);
        int lo = 1, hi = 0;
        if (tok >= 0) {
            hi = positions[t0 + tok];
            lo = window > 0 ? max(0, hi - window + 1) : 0;
        }
        row_lo[threadIdx.x] = lo; row_hi[threadIdx.x] = hi;
    }
    for (int i = threadIdx.x; i < ROWS * (D / 8); i += blockDim.x) {
        const int r = i / (D / 8), pc = (i % (D / 8)) * 8, tok = row_token(r);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tok >= 0) {
            const int h = row_head(r);
            const bf* src = pc < rank ? qa + (size_t)(t0 + tok) * qa_row + (size_t)h * qa_head + pc
                                      : q_rot + (size_t)(t0 + tok) * q_rot_row + (size_t)h * q_rot_head + pc - rank;
            if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) v = *reinterpret_cast<const uint4*>(src);
            else { bf* e = reinterpret_cast<bf*>(&v); for (int k = 0; k < 8; ++k) e[k] = src[k]; }
        }
        *reinterpret_cast<uint4*>(Qs + r * DP + pc) = v;
    }
    const int p_hi = positions[t0 + ntok - 1], p_first = positions[t0];
    const int key_lo = window > 0 ? max(0, p_first - window + 1) : 0;
    const int tiles = (p_hi - key_lo + kMmaKeys) / kMmaKeys;
    float acc[NTW][4];
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int ntw = rank / CH / 8;
    const int colw = half * (rank / CH);
    auto stage = [&](int tile, bf* dstbase) {
        const int j0 = key_lo + tile * kMmaKeys;
        const int jl = j0 + lane;
        const long long mine = jl <= p_hi ? (long long)pages[jl / page_size] * page_size + jl % page_size : -1;
        for (int jj = warp; jj < kMmaKeys; jj += 4) {
            const long long off = __shfl_sync(0xffffffffu, mine, jj);
            bf* dst = dstbase + jj * DP;
            if (off >= 0) {
                const bf* c4 = c_cache + off * rank;
                const bf* k4 = kr_cache + off * rot;
                for (int i = lane; i < rank / 8; i += 32) cp_async_16(dst + i * 8, c4 + i * 8);
                for (int i = lane; i < rot / 8; i += 32) cp_async_16(dst + rank + i * 8, k4 + i * 8);
            } else {
                for (int i = lane; i < D / 8; i += 32) reinterpret_cast<uint4*>(dst)[i] = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, Kt0);
    __syncthreads();
    const int lo0 = row_lo[rt * 16 + g], hi0 = row_hi[rt * 16 + g], lo1 = row_lo[rt * 16 + g + 8], hi1 = row_hi[rt * 16 + g + 8];
    const bf* qp = Qs + (rt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DP + (lane >> 4) * 8;
    for (int tile = 0; tile < tiles; ++tile) {
        const int j0 = key_lo + tile * kMmaKeys;
        bf* Kt = Kt0 + (tile & 1) * kMmaKeys * DP;
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();                                     // this tile has landed; the tile before is used up
        if (tile + 1 < tiles) stage(tile + 1, Kt0 + ((tile + 1) & 1) * kMmaKeys * DP);
        float s[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
        const bf* kp = Kt + (lane & 7) * DP + (lane >> 3) * 8;
        int kk = 0;
        for (; kk + 32 <= D; kk += 32) {
            uint32_t a0[4], a1[4];
            ldsm_x4(a0, qp + kk);
            ldsm_x4(a1, qp + kk + 16);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t b[4];
                ldsm_x4(b, kp + j * 8 * DP + kk);
                mma_16816(s[j], a0, b[0], b[1]);
                mma_16816(s[j], a1, b[2], b[3]);
            }
        }
        if (kk < D) {
            uint32_t a0[4];
            ldsm_x4(a0, qp + kk);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t b[2];
                ldsm_x2(b, kp + j * 8 * DP + kk);
                mma_16816(s[j], a0, b[0], b[1]);
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int jk = j0 + j * 8 + 2 * t;
            s[j][0] = (jk >= lo0 && jk <= hi0) ? s[j][0] * scale : -INFINITY;
            s[j][1] = (jk + 1 >= lo0 && jk + 1 <= hi0) ? s[j][1] * scale : -INFINITY;
            s[j][2] = (jk >= lo1 && jk <= hi1) ? s[j][2] * scale : -INFINITY;
            s[j][3] = (jk + 1 >= lo1 && jk + 1 <= hi1) ? s[j][3] * scale : -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
        const float c0 = mn0 == -INFINITY ? 1.f : expf(m[0] - mn0), c1 = mn1 == -INFINITY ? 1.f : expf(m[1] - mn1);
        m[0] = mn0; m[1] = mn1;
        uint32_t pa[4][2];                                   // the weights, rounded, as operand pieces: [key tile][row half]
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 w0 = __floats2bfloat162_rn(mn0 == -INFINITY ? 0.f : expf(s[j][0] - mn0), mn0 == -INFINITY ? 0.f : expf(s[j][1] - mn0));
            const __nv_bfloat162 w1 = __floats2bfloat162_rn(mn1 == -INFINITY ? 0.f : expf(s[j][2] - mn1), mn1 == -INFINITY ? 0.f : expf(s[j][3] - mn1));
            sum0 += __bfloat162float(w0.x) + __bfloat162float(w0.y);      // the sums take the weights as the product sees them
            sum1 += __bfloat162float(w1.x) + __bfloat162float(w1.y);
            pa[j][0] = *reinterpret_cast<const uint32_t*>(&w0);
            pa[j][1] = *reinterpret_cast<const uint32_t*>(&w1);
        }
        l[0] = l[0] * c0 + sum0;
        l[1] = l[1] * c1 + sum1;
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
            if (nt < ntw) { acc[nt][0] *= c0; acc[nt][1] *= c0; acc[nt][2] *= c1; acc[nt][3] *= c1; }
        }
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            const uint32_t a[4] = {pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0], pa[2 * ks + 1][1]};
            const bf* vp = Kt + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DP + colw + (lane >> 4) * 8;
#pragma unroll
            for (int nt = 0; nt < NTW; nt += 2) {
                if (nt + 1 < ntw) {
                    uint32_t b[4];
                    ldsm_x4_t(b, vp + nt * 8);
                    mma_16816(acc[nt], a, b[0], b[1]);
                    mma_16816(acc[nt + 1], a, b[2], b[3]);
                } else if (nt < ntw) {
                    uint32_t b[2];
                    ldsm_x2_t(b, vp + nt * 8);
                    mma_16816(acc[nt], a, b[0], b[1]);
                }
            }
        }
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        l[e] += __shfl_xor_sync(0xffffffffu, l[e], 1);
        l[e] += __shfl_xor_sync(0xffffffffu, l[e], 2);
        const int r = rt * 16 + g + 8 * e, tok = row_token(r);
        if (tok < 0) continue;
        const size_t row = (size_t)(t0 + tok) * H + row_head(r);
        if (sinks != nullptr && l[e] > 0.f) l[e] += expf(sinks[row_head(r)] - m[e]);
        const float inv = l[e] > 0.f ? 1.f / l[e] : 0.f;
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt)
            if (nt < ntw)
                *reinterpret_cast<__nv_bfloat162*>(out + row * rank + colw + nt * 8 + 2 * t) =
                    __floats2bfloat162_rn(acc[nt][2 * e] * inv, acc[nt][2 * e + 1] * inv);
    }
}

// blocks: runs of at most `wide_tokens(H, rank)` neighbouring tokens of one request, every token of the step in one.
// `rows`: 64 (a warp per row tile; rank <= 256) or 32 (two warps per row tile, half the output columns each: more,
// lighter CTAs, every score computed twice)
extern "C" int lb_latent_wide_tokens(int H, int rows) {
    return H >= 16 ? rows / 16 : rows / H;
}

extern "C" int lb_latent_attention_wide(const void* qa, long qa_row, long qa_head, const void* q_rot, long q_rot_row, long q_rot_head,
                                        const void* c_cache, const void* kr_cache, const int* block_table, int table_width,
                                        const int* token_req, const int* positions, const int* blocks, int num_blocks, void* out,
                                        int H, int rank, int rot, int page_size, float scale, int window, int rows, const float* sinks,
                                        void* stream) {
    if (num_blocks <= 0) return kOk;
    if (H <= 0 || rank <= 0 || rank % 32 || rot < 0 || rot % 16 || page_size <= 0 || window < 0) return kBadSize;
    if ((rows != 32 && rows != 64) || (rows == 64 && rank > 256)) return kBadSize;
    if (rank > 512) return kTooLarge;
    typedef __nv_bfloat16 bf;
    const int D = rank + rot;
    const size_t smem = (size_t)(rows + 2 * kMmaKeys) * (D + 8) * sizeof(bf);
    dim3 grid(num_blocks, H >= 16 ? (H + 15) / 16 : 1);
    cudaStream_t st = (cudaStream_t)stream;
#define LB_LW(NTW_, CH_) { static size_t have = 0; ensure_dynamic_smem(latent_attention_wide_kernel<NTW_, CH_>, smem, have); \
        latent_attention_wide_kernel<NTW_, CH_><<<grid, 128, smem, st>>>((const bf*)qa, qa_row, qa_head, (const bf*)q_rot, q_rot_row, \
            q_rot_head, (const bf*)c_cache, (const bf*)kr_cache, block_table, table_width, token_req, positions, blocks, (bf*)out, \
            H, rank, rot, page_size, scale, window, sinks); }
    if (rows == 64) { if (rank <= 128) LB_LW(16, 1) else LB_LW(32, 1) }
    else { if (rank <= 256) LB_LW(16, 2) else LB_LW(32, 2) }
#undef LB_LW
    return launch_status();
}

// grid (listed token blocks' rows): one CTA per (token, head) row of the step
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, int rank, int splits, const float* __restrict__ sinks, int H) {
    const size_t row = blockIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(row * splits + s) * 2]);
    if (M == -INFINITY) return;                              // a row that no block of this step owns
    float L = 0.f;
    for (int s = 0; s < splits; ++s) L += part_ml[(row * splits + s) * 2 + 1] * expf(part_ml[(row * splits + s) * 2] - M);
    if (sinks != nullptr) L += expf(sinks[row % H] - M);       // the sink joins the denominator once, here
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = part_ml[(row * splits + s) * 2];
            if (ms != -INFINITY) a += part_o[(row * splits + s) * rank + c] * expf(ms - M);
        }
        out[row * rank + c] = __float2bfloat16_rn(a / L);
    }
}

// blocks: int32 [num_blocks, 2] (first token row, tokens: neighbours of one request, at most max(1, 16 / H); -1: nothing),
// or null: every token a block of its own (num_blocks = tokens).
// Every token of the step lies in exactly one block.  part_o float32 [tokens * H, splits, rank] and part_ml float32
// [tokens * H, splits, 2]: scratch for splits > 1 (every row is written by the CTAs of its block).
extern "C" int lb_latent_attention_mma(const void* qa, long qa_row, long qa_head, const void* q_rot, long q_rot_row, long q_rot_head, const void* c_cache,
                                       const void* kr_cache, const int* block_table, int table_width, const int* token_req,
                                       const int* positions, const int* blocks, int num_blocks, void* out, float* part_o,
                                       float* part_ml, int tokens, int H, int rank, int rot, int page_size, float scale,
                                       int window, int splits, const float* sinks, void* stream) {
    if (num_blocks <= 0) return kOk;
    if (H <= 0 || rank <= 0 || rank % 32 || rot < 0 || rot % 16 || page_size <= 0 || window < 0 || splits < 1) return kBadSize;
    if (rank > 512 || splits > 65535) return kTooLarge;
    typedef __nv_bfloat16 bf;
    const int D = rank + rot;
    const size_t smem = ((size_t)(16 + 2 * kMmaKeys) * (D + 8) + 16 * (kMmaKeys + 8)) * sizeof(bf) + 64 * sizeof(float);
    dim3 grid(num_blocks, H >= 16 ? (H + 15) / 16 : 1, splits);
    cudaStream_t st = (cudaStream_t)stream;
#define LB_LA(NTW_) { static size_t have = 0; ensure_dynamic_smem(latent_attention_mma_kernel<NTW_>, smem, have); \
        latent_attention_mma_kernel<NTW_><<<grid, 128, smem, st>>>((const bf*)qa, qa_row, qa_head, (const bf*)q_rot, q_rot_row, q_rot_head, \
            (const bf*)c_cache, (const bf*)kr_cache, block_table, table_width, token_req, positions, blocks, (bf*)out, part_o, \
            part_ml, H, rank, rot, page_size, scale, window, splits, sinks); }
    if (rank <= 128) LB_LA(4) else if (rank <= 256) LB_LA(8) else LB_LA(16)
#undef LB_LA
    int rc = launch_status();
    if (rc != 0 || splits == 1) return rc;
    latent_merge_kernel<<<tokens * H, 128, 0, st>>>(part_o, part_ml, (bf*)out, rank, splits, sinks, H);
    return launch_status();
}
