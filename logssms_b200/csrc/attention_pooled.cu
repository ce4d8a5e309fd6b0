// Grouped-query attention over a sliding window of tokens plus pooled blocks behind it, with rotated values.
//
//   Query i sees the tokens j with 0 <= i - j < window and, as ONE key and value each, every block b of `pool` tokens
//   (positions b*pool .. b*pool + pool - 1) that lies wholly behind the window: b*pool + pool - 1 <= i - window, i.e.
//   the first floor((i - window + 1) / pool) blocks.  A block's key and value are the means of its tokens' cached keys
//   and values.  Tokens that have left the window and whose block is not yet complete behind it are not seen.  Tokens
//   and blocks share one softmax.
//
//   Queries and keys are rotated over neighbouring pairs (columns 2i, 2i + 1 of the first `rot` columns, angle
//   p * f_i); values are rotated the same way over ALL their columns by their own position and cached so; the
//   weighted sum of the values of query i is turned back by -i.  cos/sin come from tables [positions, n] (cos of
//   the n/2 pairs, then sin) in float32.
//
//   Two options turn the same kernels into other attentions.  `pool` = 0: there are no blocks (with a window beyond
//   every position: plain causal attention).  `slopes` (a number per query head): m_h * (i - j) is taken off the scaled
//   score of token j.  `sinks` (a number per query head): exp(sink_h) joins the softmax's denominator, with no key and no
//   value.  Without rotation tables (`v_rot` = 0) values are summed as they are cached.
//
//   pooled_prepare : per (token, head): rotate the query; rotate key and value and store them at the token's slot
//   normed_prepare : per (token, head): RMS-norm the query and the key over the head's columns with a weight each
//                    (shared by the heads), the query times 1 + coef * ln(floor((p + 1) / every) + 1) at position p;
//                    store key and value at the token's slot
//   pooled_blocks  : per token that ends a block: the means of the block's cached keys and values, stored at the
//                    block's entry of a second paged cache (one entry per `pool` tokens)
//   pooled_attention      : a warp per (token, head); a lane scores one key at a time, the lanes share the value
//                           columns; scores, softmax and sums in float32 (every dtype, every size)
//   pooled_attention_split: decoded tokens and short portions: key ranges side by side, all query heads of a key/value
//                           head in one CTA, a merge kernel behind (described at the kernel)
//   pooled_attention_tile : bfloat16 prompt portions on the tensor cores: a CTA per (run of up to 64 neighbouring tokens
//                           of a request, query head); the keys the run sees go through shared memory once for all
//                           its queries (described at the kernel)
#include "lb200/common.cuh"
using namespace lb200;

// grid (tokens, Hq + 2 * Hkv)
template <typename T>
__global__ void pooled_prepare_kernel(const T* __restrict__ qkv, long row_stride, const int* __restrict__ positions,
                                      const int* __restrict__ slot_mapping, const float* __restrict__ qk_table, int rot,
                                      const float* __restrict__ v_table, int v_rot, int table_rows, T* __restrict__ q_out,
                                      T* __restrict__ k_cache, T* __restrict__ v_cache, int Hq, int Hkv, int dim, int vdim,
                                      int write_kv) {
    const size_t t = blockIdx.x;
    int head = blockIdx.y;
    const int pos = min(max(positions[t], 0), table_rows - 1);
    const T* src;
    T* dst;
    const float* cs;
    int n, r;
    if (head < Hq) {
        src = qkv + t * row_stride + (size_t)head * dim;
        dst = q_out + (t * Hq + head) * dim;
        n = dim; r = rot; cs = qk_table + (size_t)pos * rot;
    } else {
        if (!write_kv) return;
        const long slot = slot_mapping[t];
        if (slot < 0) return;
        head -= Hq;
        if (head < Hkv) {
            src = qkv + t * row_stride + (size_t)Hq * dim + (size_t)head * dim;
            dst = k_cache + ((size_t)slot * Hkv + head) * dim;
            n = dim; r = rot; cs = qk_table + (size_t)pos * rot;
        } else {
            head -= Hkv;
            src = qkv + t * row_stride + (size_t)(Hq + Hkv) * dim + (size_t)head * vdim;
            dst = v_cache + ((size_t)slot * Hkv + head) * vdim;
            n = vdim; r = v_rot; cs = v_table + (size_t)pos * v_rot;
        }
    }
    const int half = r >> 1;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        float val = to_f32(src[c]);
        if (c < r) {
            const float partner = to_f32(src[c ^ 1]);
            const float co = cs[c >> 1], si = cs[half + (c >> 1)];
            val = (c & 1) ? val * co + partner * si : val * co - partner * si;
        }
        dst[c] = from_f32<T>(val);
    }
}

extern "C" int lb_pooled_prepare(const void* qkv, long row_stride, const int* positions, const int* slot_mapping,
                                 const float* qk_table, int rot, const float* v_table, int v_rot, int table_rows, void* q_out,
                                 void* k_cache, void* v_cache, int tokens, int Hq, int Hkv, int dim, int vdim, int write_kv,
                                 int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (Hq <= 0 || Hkv <= 0 || dim <= 0 || vdim <= 0 || rot < 0 || rot > dim || (rot & 1) || v_rot < 0 || v_rot > vdim || (v_rot & 1)
        || Hq + 2 * Hkv > 65535 || table_rows <= 0)
        return kBadSize;
    dim3 grid(tokens, Hq + 2 * Hkv);
    const int threads = max(dim, vdim) > 64 ? 128 : 64;
    LB_DISPATCH_DTYPE(dtype, pooled_prepare_kernel<T><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const T*)qkv, row_stride, positions, slot_mapping, qk_table, rot, v_table, v_rot, table_rows, (T*)q_out, (T*)k_cache,
        (T*)v_cache, Hq, Hkv, dim, vdim, write_kv));
    return launch_status();
}

// grid (tokens, Hq + 2 * Hkv); a warp per (token, head)
template <typename T>
__global__ void __launch_bounds__(32) normed_prepare_kernel(const T* __restrict__ qkv, long row_stride, const int* __restrict__ positions,
                                                            const int* __restrict__ slot_mapping, const float* __restrict__ q_weight,
                                                            const float* __restrict__ k_weight, float eps, float temp_coef, int temp_every,
                                                            T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                            int Hq, int Hkv, int dim, int vdim, int write_kv) {
    const size_t t = blockIdx.x;
    int head = blockIdx.y;
    const int lane = threadIdx.x;
    const T* src;
    T* dst;
    const float* w;
    float mult = 1.f;
    int n;
    if (head < Hq) {
        src = qkv + t * row_stride + (size_t)head * dim;
        dst = q_out + (t * Hq + head) * dim;
        n = dim; w = q_weight;
        if (temp_every > 0) mult = 1.f + temp_coef * logf((float)((max(positions[t], 0) + 1) / temp_every + 1));
    } else {
        if (!write_kv) return;
        const long slot = slot_mapping[t];
        if (slot < 0) return;
        head -= Hq;
        if (head < Hkv) {
            src = qkv + t * row_stride + (size_t)Hq * dim + (size_t)head * dim;
            dst = k_cache + ((size_t)slot * Hkv + head) * dim;
            n = dim; w = k_weight;
        } else {
            head -= Hkv;
            src = qkv + t * row_stride + (size_t)(Hq + Hkv) * dim + (size_t)head * vdim;
            dst = v_cache + ((size_t)slot * Hkv + head) * vdim;
            for (int c = lane; c < vdim; c += 32) dst[c] = src[c];
            return;
        }
    }
    float ss = 0.f;
    for (int c = lane; c < n; c += 32) { const float v = to_f32(src[c]); ss += v * v; }
    const float inv = mult / sqrtf(warp_sum(ss) / (float)n + eps);
    for (int c = lane; c < n; c += 32) dst[c] = from_f32<T>(to_f32(src[c]) * inv * w[c]);
}

// qkv: [tokens, (Hq + Hkv) * dim + Hkv * vdim] (column view allowed); q_weight, k_weight: float32 [dim]; temp_every 0: no
// query temperature
extern "C" int lb_normed_prepare(const void* qkv, long row_stride, const int* positions, const int* slot_mapping, const float* q_weight,
                                 const float* k_weight, float eps, float temp_coef, int temp_every, void* q_out, void* k_cache,
                                 void* v_cache, int tokens, int Hq, int Hkv, int dim, int vdim, int write_kv, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (Hq <= 0 || Hkv <= 0 || dim <= 0 || vdim <= 0 || Hq + 2 * Hkv > 65535 || temp_every < 0) return kBadSize;
    dim3 grid(tokens, Hq + 2 * Hkv);
    LB_DISPATCH_DTYPE(dtype, normed_prepare_kernel<T><<<grid, 32, 0, (cudaStream_t)stream>>>(
        (const T*)qkv, row_stride, positions, slot_mapping, q_weight, k_weight, eps, temp_coef, temp_every, (T*)q_out, (T*)k_cache,
        (T*)v_cache, Hq, Hkv, dim, vdim, write_kv));
    return launch_status();
}

// grid (tokens, Hkv): the token that ends a block writes the block's means
template <typename T>
__global__ void pooled_blocks_kernel(const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ kp_cache,
                                     T* __restrict__ vp_cache, const int* __restrict__ positions, const int* __restrict__ token_req,
                                     const int* __restrict__ block_table, int table_width, const int* __restrict__ pooled_slots,
                                     int Hkv, int dim, int vdim, int page_size, int pool) {
    const int t = blockIdx.x, g = blockIdx.y;
    const int pos = positions[t];
    if (pos < 0 || (pos + 1) % pool != 0) return;
    const long out_slot = pooled_slots[t];
    if (out_slot < 0) return;
    const int* pages = block_table + (size_t)token_req[t] * table_width;
    const int first = pos + 1 - pool;
    const float inv = 1.f / (float)pool;
    for (int c = threadIdx.x; c < dim + vdim; c += blockDim.x) {
        float sum = 0.f;
        for (int j = first; j <= pos; ++j) {
            const int page = pages[j / page_size];
            if (page < 0) continue;
            const size_t slot = (size_t)page * page_size + j % page_size;
            sum += c < dim ? to_f32(k_cache[(slot * Hkv + g) * dim + c]) : to_f32(v_cache[(slot * Hkv + g) * vdim + (c - dim)]);
        }
        if (c < dim) kp_cache[((size_t)out_slot * Hkv + g) * dim + c] = from_f32<T>(sum * inv);
        else vp_cache[((size_t)out_slot * Hkv + g) * vdim + (c - dim)] = from_f32<T>(sum * inv);
    }
}

extern "C" int lb_pooled_blocks(const void* k_cache, const void* v_cache, void* kp_cache, void* vp_cache, const int* positions,
                                const int* token_req, const int* block_table, int table_width, const int* pooled_slots,
                                int tokens, int Hkv, int dim, int vdim, int page_size, int pool, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (Hkv <= 0 || Hkv > 65535 || dim <= 0 || vdim <= 0 || page_size <= 0 || pool <= 0) return kBadSize;
    dim3 grid(tokens, Hkv);
    const int threads = dim + vdim > 128 ? 256 : 128;
    LB_DISPATCH_DTYPE(dtype, pooled_blocks_kernel<T><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const T*)k_cache, (const T*)v_cache, (T*)kp_cache, (T*)vp_cache, positions, token_req, block_table, table_width,
        pooled_slots, Hkv, dim, vdim, page_size, pool));
    return launch_status();
}

// ------------------------------------------------------------------------------------------------ attention, a warp per row
constexpr int kWarps = 4;            // (token, head) rows of a CTA: neighbouring heads of one token
constexpr int kMaxValueRegs = 8;     // value columns per lane: vdim <= 256

// the cache row of key number `kk` of a query: the first `blocks` keys are pooled blocks, the others the window's tokens
__device__ __forceinline__ long key_row(int kk, int blocks, int first, const int* __restrict__ pages, const int* __restrict__ pooled_pages,
                                        int page_size, bool& pooled) {
    pooled = kk < blocks;
    const int e = pooled ? kk : first + (kk - blocks);
    const int page = (pooled ? pooled_pages : pages)[e / page_size];
    return page < 0 ? -1 : (long)page * page_size + e % page_size;
}

// blocks that lie wholly behind the window of position i (none without pooling)
__device__ __forceinline__ int blocks_behind(int i, int window, int pool) {
    return pool > 0 ? max(0, (i - window + 1) / pool) : 0;
}

// what two options add to a softmax: a slope per head on the distance to a token, a sink per head in the denominator
struct ScoreExtras {
    const float* slopes;      // [Hq] or null
    const float* sinks;       // [Hq] or null
};

// (maximum, sum, weighted values scaled by `f`) of a softmax once the sink has joined it
__device__ __forceinline__ void join_sink(float sink, float& m, float& l, float& f) {
    const float m_new = fmaxf(m, sink);
    f = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * f + expf(sink - m_new);
    m = m_new;
}

// grid (tokens, ceil(Hq / kWarps)); dynamic shared memory: kWarps * dim floats (the scaled queries)
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) pooled_attention_kernel(
        const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, const T* __restrict__ kp_cache,
        const T* __restrict__ vp_cache, const int* __restrict__ block_table, int table_width, const int* __restrict__ pooled_table,
        int pooled_width, const int* __restrict__ token_req, const int* __restrict__ positions, const int* __restrict__ token_list,
        const float* __restrict__ v_table, int v_rot, int table_rows, T* __restrict__ out, int Hq, int Hkv, int dim, int vdim,
        int page_size, float scale, int window, int pool, ScoreExtras extras) {
    extern __shared__ float q_s[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = token_list != nullptr ? token_list[blockIdx.x] : blockIdx.x;
    const int head = blockIdx.y * kWarps + warp;
    if (t < 0 || head >= Hq) return;
    const int g = head / (Hq / Hkv);
    const int pos = positions[t];
    float* qs = q_s + warp * dim;
    for (int c = lane; c < dim; c += 32) qs[c] = to_f32(q[((size_t)t * Hq + head) * dim + c]) * scale;
    __syncwarp();
    const int* pages = block_table + (size_t)token_req[t] * table_width;
    const int* pooled_pages = pooled_table + (size_t)token_req[t] * pooled_width;
    const int first = max(0, pos - window + 1);
    const int blocks = blocks_behind(pos, window, pool);
    const int keys = blocks + (pos - first + 1);
    const float slope = extras.slopes != nullptr ? extras.slopes[head] : 0.f;
    float m = -INFINITY, l = 0.f, acc[kMaxValueRegs];
#pragma unroll
    for (int r = 0; r < kMaxValueRegs; ++r) acc[r] = 0.f;
    for (int k0 = 0; k0 < keys; k0 += 32) {
        const int kk = k0 + lane;
        float s = -INFINITY;
        long row = -1;
        bool pooled = false;
        if (kk < keys) {
            row = key_row(kk, blocks, first, pages, pooled_pages, page_size, pooled);
            if (row >= 0) {
                const T* kr = (pooled ? kp_cache : k_cache) + ((size_t)row * Hkv + g) * dim;
                float a0 = 0.f, a1 = 0.f;
                int c = 0;
                for (; c + 2 <= dim; c += 2) { a0 += qs[c] * to_f32(kr[c]); a1 += qs[c + 1] * to_f32(kr[c + 1]); }
                if (c < dim) a0 += qs[c] * to_f32(kr[c]);
                s = a0 + a1;
                if (!pooled) s -= slope * (float)(pos - (first + kk - blocks));
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;
        const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
        const float p = s == -INFINITY ? 0.f : expf(s - m_new);
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int r = 0; r < kMaxValueRegs; ++r) acc[r] *= corr;
        const int n = min(32, keys - k0);
        for (int j = 0; j < n; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long rj = __shfl_sync(0xffffffffu, row, j);
            const bool pooled_j = (k0 + j) < blocks;
            if (rj < 0 || pj == 0.f) continue;
            const T* vr = (pooled_j ? vp_cache : v_cache) + ((size_t)rj * Hkv + g) * vdim;
#pragma unroll
            for (int r = 0; r < kMaxValueRegs; ++r) {
                const int c = lane + 32 * r;
                if (c < vdim) acc[r] += pj * to_f32(vr[c]);
            }
        }
    }
    if (extras.sinks != nullptr) {
        float f;
        join_sink(extras.sinks[head], m, l, f);
#pragma unroll
        for (int r = 0; r < kMaxValueRegs; ++r) acc[r] *= f;
    }
    // the summed values, turned back by the query's position (pairs of neighbouring columns: neighbouring lanes)
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
    const float* cs = v_table + (size_t)min(max(pos, 0), table_rows - 1) * v_rot;
    const int half = v_rot >> 1;
#pragma unroll
    for (int r = 0; r < kMaxValueRegs; ++r) {
        const int c = lane + 32 * r;
        const float own = acc[r] * inv_l;
        const float partner = __shfl_xor_sync(0xffffffffu, own, 1);
        if (c < vdim) {
            float val = own;
            if (c < v_rot) {
                const float co = cs[c >> 1], si = cs[half + (c >> 1)];
                val = (c & 1) ? own * co - partner * si : own * co + partner * si;
            }
            out[((size_t)t * Hq + head) * vdim + c] = from_f32<T>(val);
        }
    }
}

extern "C" int lb_pooled_attention(const void* q, const void* k_cache, const void* v_cache, const void* kp_cache,
                                   const void* vp_cache, const int* block_table, int table_width, const int* pooled_table,
                                   int pooled_width, const int* token_req, const int* positions, const int* token_list,
                                   int num_tokens, const float* v_table, int v_rot, int table_rows, void* out, int Hq, int Hkv,
                                   int dim, int vdim, int page_size, float scale, int window, int pool, const float* slopes,
                                   const float* sinks, int dtype, void* stream) {
    if (num_tokens <= 0) return kOk;
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || dim <= 0 || vdim <= 0 || page_size <= 0 || window <= 0 || pool < 0 || (v_rot & 1)
        || v_rot > vdim || table_rows <= 0)
        return kBadSize;
    if (vdim > 32 * kMaxValueRegs || (size_t)kWarps * dim * sizeof(float) > 48 * 1024) return kTooLarge;
    dim3 grid(num_tokens, (Hq + kWarps - 1) / kWarps);
    LB_DISPATCH_DTYPE(dtype, pooled_attention_kernel<T><<<grid, kWarps * 32, (size_t)kWarps * dim * sizeof(float), (cudaStream_t)stream>>>(
        (const T*)q, (const T*)k_cache, (const T*)v_cache, (const T*)kp_cache, (const T*)vp_cache, block_table, table_width,
        pooled_table, pooled_width, token_req, positions, token_list, v_table, v_rot, table_rows, (T*)out, Hq, Hkv, dim, vdim,
        page_size, scale, window, pool, ScoreExtras{slopes, sinks}));
    return launch_status();
}

// ------------------------------------------------------------------------------------------------ decoded tokens: key ranges side by side
// A CTA takes one token, one key/value head and one of `splits` ranges of the token's keys (pooled blocks first, then
// the window's tokens) for ALL query heads of that key/value head: a lane scores one key at a time for every head
// (the key row is read once, in 16-byte pieces where the size allows), then the lanes share the value columns of
// the warp's 32 keys.  The four warps' partial (maximum, sum, weighted values) meet in shared memory and go to a
// scratch buffer; `pooled_merge` joins the ranges, divides, turns the values back and stores.  All float32.
constexpr int kSplitWarps = 4;
constexpr int kSplitValueRegs = 4;        // value columns per lane: vdim <= 128

template <typename T, int kPer>
__device__ __forceinline__ void score_row(const T* __restrict__ kr, const float* __restrict__ qs, int dim, float (&s)[kPer]) {
    for (int c = 0; c < dim; ++c) {
        const float kv = to_f32(kr[c]);
#pragma unroll
        for (int h = 0; h < kPer; ++h) s[h] += qs[h * dim + c] * kv;
    }
}
template <int kPer>
__device__ __forceinline__ void score_row_vec(const __nv_bfloat16* __restrict__ kr, const float* __restrict__ qs, int dim, float (&s)[kPer]) {
    for (int c = 0; c < dim; c += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(kr + c);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float kv[8];
#pragma unroll
        for (int x = 0; x < 4; ++x) { const float2 f = __bfloat1622float2(p2[x]); kv[2 * x] = f.x; kv[2 * x + 1] = f.y; }
#pragma unroll
        for (int h = 0; h < kPer; ++h) {
            const float4 q0 = *reinterpret_cast<const float4*>(qs + h * dim + c), q1 = *reinterpret_cast<const float4*>(qs + h * dim + c + 4);
            s[h] += q0.x * kv[0] + q0.y * kv[1] + q0.z * kv[2] + q0.w * kv[3] + q1.x * kv[4] + q1.y * kv[5] + q1.z * kv[6] + q1.w * kv[7];
        }
    }
}

// grid (tokens, Hkv * ceil(per / kPer), splits); dynamic shared memory: kPer * dim floats (queries) + the warps' partial results
// partial: float [tokens, Hq, splits, vdim + 2] (maximum, sum, weighted values)
template <typename T, int kPer>
__global__ void __launch_bounds__(kSplitWarps * 32) pooled_attention_split_kernel(
        const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, const T* __restrict__ kp_cache,
        const T* __restrict__ vp_cache, const int* __restrict__ block_table, int table_width, const int* __restrict__ pooled_table,
        int pooled_width, const int* __restrict__ token_req, const int* __restrict__ positions, const int* __restrict__ token_list,
        float* __restrict__ partial, int Hq, int Hkv, int dim, int vdim, int page_size, float scale, int window, int pool, int splits,
        ScoreExtras extras) {
    extern __shared__ __align__(16) float split_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slot = blockIdx.x;                                   // row of the scratch buffer
    const int t = token_list != nullptr ? token_list[slot] : slot;
    if (t < 0) return;
    const int per = Hq / Hkv, groups = (per + kPer - 1) / kPer;
    const int g = blockIdx.y / groups, h0 = g * per + (blockIdx.y % groups) * kPer;
    const int nh = min(kPer, g * per + per - h0);                  // query heads of this CTA
    const int split = blockIdx.z;
    float* qs = split_smem;                                        // [kPer][dim]
    float* part = split_smem + kPer * dim;                         // [warps][kPer][vdim + 2]
    for (int i = threadIdx.x; i < kPer * dim; i += blockDim.x) {
        const int h = i / dim, c = i % dim;
        qs[i] = h < nh ? to_f32(q[((size_t)t * Hq + h0 + h) * dim + c]) * scale : 0.f;
    }
    __syncthreads();
    const int pos = positions[t];
    const int* pages = block_table + (size_t)token_req[t] * table_width;
    const int* pooled_pages = pooled_table + (size_t)token_req[t] * pooled_width;
    const int first = max(0, pos - window + 1);
    const int blocks = blocks_behind(pos, window, pool);
    const int keys = blocks + (pos - first + 1);
    float slope[kPer];
#pragma unroll
    for (int h = 0; h < kPer; ++h) slope[h] = (extras.slopes != nullptr && h < nh) ? extras.slopes[h0 + h] : 0.f;
    const int chunk = ((keys + splits - 1) / splits + 31) / 32 * 32;
    const int k_begin = split * chunk, k_end = min(keys, k_begin + chunk);
    const bool vec = sizeof(T) == 2 && dim % 8 == 0;
    float m[kPer], l[kPer], acc[kPer][kSplitValueRegs];
#pragma unroll
    for (int h = 0; h < kPer; ++h) {
        m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
        for (int r = 0; r < kSplitValueRegs; ++r) acc[h][r] = 0.f;
    }
    for (int k0 = k_begin + warp * 32; k0 < k_end; k0 += kSplitWarps * 32) {
        const int kk = k0 + lane;
        float s[kPer];
#pragma unroll
        for (int h = 0; h < kPer; ++h) s[h] = 0.f;
        long row = -1;
        bool pooled = false;
        if (kk < k_end) row = key_row(kk, blocks, first, pages, pooled_pages, page_size, pooled);
        if (row >= 0) {
            const T* kr = (pooled ? kp_cache : k_cache) + ((size_t)row * Hkv + g) * dim;
            if (vec) score_row_vec<kPer>(reinterpret_cast<const __nv_bfloat16*>(kr), qs, dim, s);
            else score_row<T, kPer>(kr, qs, dim, s);
            if (!pooled) {
                const float dist = (float)(pos - (first + kk - blocks));
#pragma unroll
                for (int h = 0; h < kPer; ++h) s[h] -= slope[h] * dist;
            }
        }
        float p[kPer];
#pragma unroll
        for (int h = 0; h < kPer; ++h) {
            const float sv = row >= 0 ? s[h] : -INFINITY;
            const float m_new = fmaxf(m[h], warp_max(sv));
            const float corr = (m[h] == -INFINITY) ? 0.f : expf(m[h] - m_new);
            p[h] = (sv == -INFINITY) ? 0.f : expf(sv - m_new);
            l[h] = l[h] * corr + warp_sum(p[h]);
            m[h] = m_new;
#pragma unroll
            for (int r = 0; r < kSplitValueRegs; ++r) acc[h][r] *= corr;
        }
        const int n = min(32, k_end - k0);
        for (int j = 0; j < n; ++j) {
            const long rj = __shfl_sync(0xffffffffu, row, j);
            if (rj < 0) continue;
            const T* vr = ((k0 + j) < blocks ? vp_cache : v_cache) + ((size_t)rj * Hkv + g) * vdim;
            float vv[kSplitValueRegs];
#pragma unroll
            for (int r = 0; r < kSplitValueRegs; ++r) { const int c = lane + 32 * r; vv[r] = c < vdim ? to_f32(vr[c]) : 0.f; }
#pragma unroll
            for (int h = 0; h < kPer; ++h) {
                const float pj = __shfl_sync(0xffffffffu, p[h], j);
#pragma unroll
                for (int r = 0; r < kSplitValueRegs; ++r) acc[h][r] += pj * vv[r];
            }
        }
    }
    // the warps' partial results meet: warp 0 joins them
    const int stride = vdim + 2;
#pragma unroll
    for (int h = 0; h < kPer; ++h) {
        float* dst = part + ((size_t)warp * kPer + h) * stride;
        if (lane == 0) { dst[0] = m[h]; dst[1] = l[h]; }
#pragma unroll
        for (int r = 0; r < kSplitValueRegs; ++r) { const int c = lane + 32 * r; if (c < vdim) dst[2 + c] = acc[h][r]; }
    }
    __syncthreads();
    for (int h = warp; h < nh; h += kSplitWarps) {
        float mm = -INFINITY;
        for (int w = 0; w < kSplitWarps; ++w) mm = fmaxf(mm, part[((size_t)w * kPer + h) * stride]);
        float ll = 0.f, o[kSplitValueRegs];
#pragma unroll
        for (int r = 0; r < kSplitValueRegs; ++r) o[r] = 0.f;
        for (int w = 0; w < kSplitWarps; ++w) {
            const float* src = part + ((size_t)w * kPer + h) * stride;
            const float f = (src[0] == -INFINITY) ? 0.f : expf(src[0] - mm);
            ll += f * src[1];
#pragma unroll
            for (int r = 0; r < kSplitValueRegs; ++r) { const int c = lane + 32 * r; if (c < vdim) o[r] += f * src[2 + c]; }
        }
        float* dst = partial + (((size_t)slot * Hq + h0 + h) * splits + split) * stride;
        if (lane == 0) { dst[0] = mm; dst[1] = ll; }
#pragma unroll
        for (int r = 0; r < kSplitValueRegs; ++r) { const int c = lane + 32 * r; if (c < vdim) dst[2 + c] = o[r]; }
    }
}

// grid (tokens, Hq), a warp: joins the ranges, divides by the sum, turns the values back by the query's position
template <typename T>
__global__ void __launch_bounds__(32) pooled_merge_kernel(const float* __restrict__ partial, const int* __restrict__ positions,
                                                          const int* __restrict__ token_list, const float* __restrict__ v_table, int v_rot,
                                                          int table_rows, T* __restrict__ out, int Hq, int vdim, int splits,
                                                          const float* __restrict__ sinks) {
    const int lane = threadIdx.x, slot = blockIdx.x, head = blockIdx.y;
    const int t = token_list != nullptr ? token_list[slot] : slot;
    if (t < 0) return;
    const int stride = vdim + 2;
    const float* src0 = partial + ((size_t)slot * Hq + head) * splits * stride;
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, src0[(size_t)s * stride]);
    if (sinks != nullptr) mm = fmaxf(mm, sinks[head]);
    float ll = sinks != nullptr ? expf(sinks[head] - mm) : 0.f, o[kSplitValueRegs];
#pragma unroll
    for (int r = 0; r < kSplitValueRegs; ++r) o[r] = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float* src = src0 + (size_t)s * stride;
        const float f = (src[0] == -INFINITY) ? 0.f : expf(src[0] - mm);
        ll += f * src[1];
#pragma unroll
        for (int r = 0; r < kSplitValueRegs; ++r) { const int c = lane + 32 * r; if (c < vdim) o[r] += f * src[2 + c]; }
    }
    const float inv_l = ll > 0.f ? 1.f / ll : 0.f;
    const float* cs = v_table + (size_t)min(max(positions[t], 0), table_rows - 1) * v_rot;
    const int half = v_rot >> 1;
#pragma unroll
    for (int r = 0; r < kSplitValueRegs; ++r) {
        const int c = lane + 32 * r;
        const float own = o[r] * inv_l;
        const float partner = __shfl_xor_sync(0xffffffffu, own, 1);
        if (c < vdim) {
            float val = own;
            if (c < v_rot) {
                const float co = cs[c >> 1], si = cs[half + (c >> 1)];
                val = (c & 1) ? own * co - partner * si : own * co + partner * si;
            }
            out[((size_t)t * Hq + head) * vdim + c] = from_f32<T>(val);
        }
    }
}

template <typename T, int kPer>
static int launch_split(const void* q, const void* k_cache, const void* v_cache, const void* kp_cache, const void* vp_cache,
                        const int* block_table, int table_width, const int* pooled_table, int pooled_width, const int* token_req,
                        const int* positions, const int* token_list, int num_tokens, float* partial, int Hq, int Hkv, int dim, int vdim,
                        int page_size, float scale, int window, int pool, int splits, ScoreExtras extras, void* stream) {
    const size_t smem = ((size_t)kPer * dim + (size_t)kSplitWarps * kPer * (vdim + 2)) * sizeof(float);
    static size_t have = 0;
    ensure_dynamic_smem(pooled_attention_split_kernel<T, kPer>, smem, have);
    const int per = Hq / Hkv;
    dim3 grid(num_tokens, Hkv * ((per + kPer - 1) / kPer), splits);
    pooled_attention_split_kernel<T, kPer><<<grid, kSplitWarps * 32, smem, (cudaStream_t)stream>>>(
        (const T*)q, (const T*)k_cache, (const T*)v_cache, (const T*)kp_cache, (const T*)vp_cache, block_table, table_width,
        pooled_table, pooled_width, token_req, positions, token_list, partial, Hq, Hkv, dim, vdim, page_size, scale, window, pool, splits,
        extras);
    return launch_status();
}

// partial: float32 scratch of num_tokens * Hq * splits * (vdim + 2); vdim <= 128; dim a multiple of 4
extern "C" int lb_pooled_attention_split(const void* q, const void* k_cache, const void* v_cache, const void* kp_cache,
                                         const void* vp_cache, const int* block_table, int table_width, const int* pooled_table,
                                         int pooled_width, const int* token_req, const int* positions, const int* token_list,
                                         int num_tokens, const float* v_table, int v_rot, int table_rows, float* partial, void* out,
                                         int Hq, int Hkv, int dim, int vdim, int page_size, float scale, int window, int pool,
                                         int splits, const float* slopes, const float* sinks, int dtype, void* stream) {
    if (num_tokens <= 0) return kOk;
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || dim <= 0 || dim % 4 || vdim <= 0 || page_size <= 0 || window <= 0 || pool < 0 || (v_rot & 1)
        || v_rot > vdim || table_rows <= 0 || splits <= 0 || splits > 65535 || Hq > 65535)
        return kBadSize;
    if (vdim > 32 * kSplitValueRegs || dim > 1024) return kTooLarge;
    const int per = Hq / Hkv;
    int code;
#define LB_SPLIT(PER) LB_DISPATCH_DTYPE(dtype, code = (launch_split<T, PER>(q, k_cache, v_cache, kp_cache, vp_cache, block_table, table_width, \
        pooled_table, pooled_width, token_req, positions, token_list, num_tokens, partial, Hq, Hkv, dim, vdim, page_size, scale, window, pool, splits, \
        ScoreExtras{slopes, nullptr}, stream)))
    if (per == 1) { LB_SPLIT(1); } else if (per == 2) { LB_SPLIT(2); } else { LB_SPLIT(4); }
#undef LB_SPLIT
    if (code != 0) return code;
    dim3 grid(num_tokens, Hq);
    LB_DISPATCH_DTYPE(dtype, pooled_merge_kernel<T><<<grid, 32, 0, (cudaStream_t)stream>>>(partial, positions, token_list, v_table, v_rot,
                                                                                           table_rows, (T*)out, Hq, vdim, splits, sinks));
    return launch_status();
}

// ------------------------------------------------------------------------------------------------ prompt portions on the tensor cores
// A CTA takes one query head and a run of up to kTileQ neighbouring tokens of one request (four warps of 16 query rows).
// The keys the run sees - the pooled blocks behind the LAST query's window, then the tokens from the FIRST query's
// window to the last query - go through shared memory in chunks of kTileK, each row masked per query.  S = Q K^T and
// P V are `mma.sync` m16n8k16 products of bfloat16 operands with float32 accumulators; scores, maxima, weights and
// sums are float32.  The chunks alternate between two buffers: the next one travels by `cp.async` while this one is used.  A weight p enters P V as the two bfloat16 terms hi = bf16(p), lo = bf16(p - hi) (two products
// into the same accumulator), so it is applied to 16 bits and more, not rounded to 8.
constexpr int kTileQ = 64, kTileK = 64, kTileThreads = 128;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// grid (tiles, Hq); tiles: int32 [n, 2] (request, first token of the run within its portion), request -1: no work
template <int kDimSteps, int kValueTiles>
__global__ void __launch_bounds__(kTileThreads) pooled_attention_tile_kernel(
        const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
        const __nv_bfloat16* __restrict__ kp_cache, const __nv_bfloat16* __restrict__ vp_cache, const int* __restrict__ block_table,
        int table_width, const int* __restrict__ pooled_table, int pooled_width, const int* __restrict__ cu,
        const int* __restrict__ start_pos, const int* __restrict__ tiles, const float* __restrict__ v_table, int v_rot,
        int table_rows, __nv_bfloat16* __restrict__ out, int Hq, int Hkv, int dim, int vdim, int page_size, float scale,
        int window, int pool, float* __restrict__ partial, int splits, ScoreExtras extras) {
    extern __shared__ __align__(16) unsigned char tile_smem[];
    const int b = tiles[2 * blockIdx.x];
    if (b < 0) return;
    const int t0 = tiles[2 * blockIdx.x + 1];
    const int head = blockIdx.y, g = head / (Hq / Hkv);
    const int n_q = min(kTileQ, cu[b + 1] - cu[b] - t0);
    const int row0 = cu[b] + t0, pos0 = start_pos[b] + t0;
    const int i_last = pos0 + n_q - 1;
    const int first = max(0, pos0 - window + 1);                    // the oldest token any query of the run sees
    const int blocks = blocks_behind(i_last, window, pool);         // the blocks the last query sees
    const float slope = extras.slopes != nullptr ? extras.slopes[head] : 0.f;
    const int keys = blocks + (i_last - first + 1);
    const int k_stride = dim + 8, v_stride = vdim + 8;              // elements; the pad staggers the banks
    // two buffers of a chunk's keys and values: the next chunk travels (cp.async) while this one is multiplied
    __nv_bfloat16* Ks0 = reinterpret_cast<__nv_bfloat16*>(tile_smem);
    __nv_bfloat16* Vs0 = Ks0 + 2 * kTileK * k_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gq = lane >> 2, tq = lane & 3;
    const int dsteps = dim / 16, vtiles = vdim / 8;
    const int* pages = block_table + (size_t)b * table_width;
    const int* pooled_pages = pooled_table + (size_t)b * pooled_width;

    // this thread's two query rows and their A fragments
    const int r_lo = warp * 16 + gq, r_hi = r_lo + 8;
    const int i_lo = pos0 + r_lo, i_hi = pos0 + r_hi;
    uint32_t qa[kDimSteps][4];
#pragma unroll
    for (int ks = 0; ks < kDimSteps; ++ks) {
#pragma unroll
        for (int x = 0; x < 4; ++x) qa[ks][x] = 0u;
        if (ks < dsteps) {
            const int c = ks * 16 + 2 * tq;
            if (r_lo < n_q) {
                const __nv_bfloat16* qr = q + ((size_t)(row0 + r_lo) * Hq + head) * dim;
                qa[ks][0] = *reinterpret_cast<const uint32_t*>(qr + c);
                qa[ks][2] = *reinterpret_cast<const uint32_t*>(qr + c + 8);
            }
            if (r_hi < n_q) {
                const __nv_bfloat16* qr = q + ((size_t)(row0 + r_hi) * Hq + head) * dim;
                qa[ks][1] = *reinterpret_cast<const uint32_t*>(qr + c);
                qa[ks][3] = *reinterpret_cast<const uint32_t*>(qr + c + 8);
            }
        }
    }
    const int nb_lo = blocks_behind(i_lo, window, pool), nb_hi = blocks_behind(i_hi, window, pool);
    // what the warp's 16 rows can see at all: a chunk wholly outside is skipped
    const int iw0 = pos0 + warp * 16, iw1 = min(iw0 + 15, i_last);
    const int nb_warp = blocks_behind(iw1, window, pool);
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    float o[kValueTiles][4];
#pragma unroll
    for (int n = 0; n < kValueTiles; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    // thread 2r copies the key row of the chunk's key r, thread 2r + 1 its value row, in 16-byte pieces; a key that does
    // not exist (behind the last one, a page that is not there) becomes a row of zeros
    auto prefetch = [&](int k0, int buf) {
        const int r = threadIdx.x >> 1;
        const bool is_v = threadIdx.x & 1;
        const int kk = k0 + r;
        long row = -1;
        bool pooled = false;
        if (kk < keys) row = key_row(kk, blocks, first, pages, pooled_pages, page_size, pooled);
        const int n = is_v ? vdim : dim;
        const __nv_bfloat16* src = is_v ? (pooled ? vp_cache : v_cache) : (pooled ? kp_cache : k_cache);
        if (row >= 0) src += ((size_t)row * Hkv + g) * n;
        __nv_bfloat16* dst = is_v ? Vs0 + ((size_t)buf * kTileK + r) * v_stride : Ks0 + ((size_t)buf * kTileK + r) * k_stride;
        const uint32_t dst_addr = (uint32_t)__cvta_generic_to_shared(dst);
        const int bytes = row >= 0 ? 16 : 0;
        for (int pc = 0; pc < n / 8; ++pc)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_addr + pc * 16), "l"(src + (row >= 0 ? pc * 8 : 0)), "r"(bytes));
        asm volatile("cp.async.commit_group;");
    };
    // with `splits` > 1 (few tiles: a lone prompt) the CTAs blockIdx.z = 0 .. splits - 1 share the run's chunks; each
    // leaves its (maximum, sum, weighted values) in `partial`, and `pooled_merge` joins them
    const int chunks_all = (keys + kTileK - 1) / kTileK, chunks_per = (chunks_all + splits - 1) / splits;
    const int k_first = min(keys, (int)blockIdx.z * chunks_per * kTileK), k_last = min(keys, k_first + chunks_per * kTileK);
    if (k_first < k_last) prefetch(k_first, 0);
    for (int k0 = k_first, it = 0; k0 < k_last; k0 += kTileK, ++it) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                             // this chunk has landed; the chunk before is consumed by every warp
        if (k0 + kTileK < k_last) prefetch(k0 + kTileK, (it + 1) & 1);
        const __nv_bfloat16* Ks = Ks0 + (size_t)(it & 1) * kTileK * k_stride;
        const __nv_bfloat16* Vs = Vs0 + (size_t)(it & 1) * kTileK * v_stride;
        // is any key of the chunk visible to any row of this warp?
        {
            bool any = false;
            const int c_last = min(k0 + kTileK, keys) - 1;
            if (k0 < blocks && k0 < nb_warp) any = true;
            if (c_last >= blocks) {
                const int ja = first + max(k0, blocks) - blocks, jb = first + c_last - blocks;
                if (jb > iw0 - window && ja <= iw1) any = true;
            }
            if (!any || iw0 > i_last) continue;
        }
        // S = Q K^T
        float sc[kTileK / 8][4];
#pragma unroll
        for (int n = 0; n < kTileK / 8; ++n) {
            sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
            const __nv_bfloat16* kr = Ks + (n * 8 + gq) * k_stride + 2 * tq;
#pragma unroll
            for (int ks = 0; ks < kDimSteps; ++ks)
                if (ks < dsteps)
                    mma_bf16(sc[n], qa[ks], *reinterpret_cast<const uint32_t*>(kr + ks * 16), *reinterpret_cast<const uint32_t*>(kr + ks * 16 + 8));
        }
        // mask, scale, running maxima
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int n = 0; n < kTileK / 8; ++n) {
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int kk = k0 + n * 8 + 2 * tq + (x & 1);
                const bool hi = x >= 2;
                const int i = hi ? i_hi : i_lo;
                bool seen = kk < keys && (hi ? r_hi : r_lo) < n_q;
                float bias = 0.f;
                if (seen) {
                    if (kk < blocks) seen = kk < (hi ? nb_hi : nb_lo);
                    else { const int j = first + kk - blocks; seen = j <= i && j > i - window; bias = slope * (float)(i - j); }
                }
                const float v = seen ? sc[n][x] * scale - bias : -INFINITY;
                sc[n][x] = v;
                if (hi) mx_hi = fmaxf(mx_hi, v); else mx_lo = fmaxf(mx_lo, v);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1)); mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1)); mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float c_lo = (m_lo == -INFINITY) ? 0.f : expf(m_lo - mn_lo), c_hi = (m_hi == -INFINITY) ? 0.f : expf(m_hi - mn_hi);
        m_lo = mn_lo; m_hi = mn_hi;
        float s_lo = 0.f, s_hi = 0.f;
#pragma unroll
        for (int n = 0; n < kTileK / 8; ++n) {
            sc[n][0] = (sc[n][0] == -INFINITY) ? 0.f : expf(sc[n][0] - mn_lo);
            sc[n][1] = (sc[n][1] == -INFINITY) ? 0.f : expf(sc[n][1] - mn_lo);
            sc[n][2] = (sc[n][2] == -INFINITY) ? 0.f : expf(sc[n][2] - mn_hi);
            sc[n][3] = (sc[n][3] == -INFINITY) ? 0.f : expf(sc[n][3] - mn_hi);
            s_lo += sc[n][0] + sc[n][1];
            s_hi += sc[n][2] + sc[n][3];
        }
        s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 1); s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 2);
        s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 1); s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 2);
        l_lo = l_lo * c_lo + s_lo;
        l_hi = l_hi * c_hi + s_hi;
#pragma unroll
        for (int n = 0; n < kValueTiles; ++n) { o[n][0] *= c_lo; o[n][1] *= c_lo; o[n][2] *= c_hi; o[n][3] *= c_hi; }
        // O += P V, P in two bfloat16 terms
#pragma unroll
        for (int kstep = 0; kstep < kTileK / 16; ++kstep) {
            uint32_t ph[4], pl[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const float a = sc[2 * kstep + (x >> 1)][(x & 1) * 2], c = sc[2 * kstep + (x >> 1)][(x & 1) * 2 + 1];
                const float ah = __bfloat162float(__float2bfloat16_rn(a)), ch = __bfloat162float(__float2bfloat16_rn(c));
                ph[x] = pack_bf16(ah, ch);
                pl[x] = pack_bf16(a - ah, c - ch);
            }
            const uint32_t v_addr = (uint32_t)__cvta_generic_to_shared(Vs + (kstep * 16 + (lane & 15)) * v_stride);
#pragma unroll
            for (int n = 0; n < kValueTiles; ++n) {
                if (n < vtiles) {
                    uint32_t b0, b1;
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(v_addr + n * 16));
                    mma_bf16(o[n], ph, b0, b1);
                    mma_bf16(o[n], pl, b0, b1);
                }
            }
        }
    }
    if (partial != nullptr) {
        const int stride = vdim + 2;
        float* p_lo = partial + (((size_t)(row0 + r_lo) * Hq + head) * splits + blockIdx.z) * stride;
        float* p_hi = partial + (((size_t)(row0 + r_hi) * Hq + head) * splits + blockIdx.z) * stride;
        if (tq == 0 && r_lo < n_q) { p_lo[0] = m_lo; p_lo[1] = l_lo; }
        if (tq == 0 && r_hi < n_q) { p_hi[0] = m_hi; p_hi[1] = l_hi; }
#pragma unroll
        for (int n = 0; n < kValueTiles; ++n) {
            if (n >= vtiles) continue;
            const int c = n * 8 + 2 * tq;
            if (r_lo < n_q) { p_lo[2 + c] = o[n][0]; p_lo[3 + c] = o[n][1]; }
            if (r_hi < n_q) { p_hi[2 + c] = o[n][2]; p_hi[3 + c] = o[n][3]; }
        }
        return;
    }
    if (extras.sinks != nullptr) {
        float f_lo, f_hi;
        join_sink(extras.sinks[head], m_lo, l_lo, f_lo);
        join_sink(extras.sinks[head], m_hi, l_hi, f_hi);
#pragma unroll
        for (int n = 0; n < kValueTiles; ++n) { o[n][0] *= f_lo; o[n][1] *= f_lo; o[n][2] *= f_hi; o[n][3] *= f_hi; }
    }
    // weights' sums, the turn back by the query's position, the store
    const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
    const int half = v_rot >> 1;
    const float* cs_lo = v_table + (size_t)min(max(i_lo, 0), table_rows - 1) * v_rot;
    const float* cs_hi = v_table + (size_t)min(max(i_hi, 0), table_rows - 1) * v_rot;
#pragma unroll
    for (int n = 0; n < kValueTiles; ++n) {
        if (n >= vtiles) continue;
        const int c = n * 8 + 2 * tq;
        if (r_lo < n_q) {
            float u = o[n][0] * inv_lo, v = o[n][1] * inv_lo;
            if (c < v_rot) { const float co = cs_lo[c >> 1], si = cs_lo[half + (c >> 1)]; const float u2 = u * co + v * si; v = v * co - u * si; u = u2; }
            *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r_lo) * Hq + head) * vdim + c) = pack_bf16(u, v);
        }
        if (r_hi < n_q) {
            float u = o[n][2] * inv_hi, v = o[n][3] * inv_hi;
            if (c < v_rot) { const float co = cs_hi[c >> 1], si = cs_hi[half + (c >> 1)]; const float u2 = u * co + v * si; v = v * co - u * si; u = u2; }
            *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r_hi) * Hq + head) * vdim + c) = pack_bf16(u, v);
        }
    }
}

template <int kDimSteps, int kValueTiles>
static int launch_tile(const void* q, const void* k_cache, const void* v_cache, const void* kp_cache, const void* vp_cache,
                       const int* block_table, int table_width, const int* pooled_table, int pooled_width, const int* cu,
                       const int* start_pos, const int* tiles, int num_tiles, const float* v_table, int v_rot, int table_rows,
                       void* out, int Hq, int Hkv, int dim, int vdim, int page_size, float scale, int window, int pool,
                       float* partial, int splits, ScoreExtras extras, void* stream) {
    const size_t smem = (size_t)2 * kTileK * ((dim + 8) + (vdim + 8)) * sizeof(__nv_bfloat16);
    static size_t have = 0;
    ensure_dynamic_smem(pooled_attention_tile_kernel<kDimSteps, kValueTiles>, smem, have);
    dim3 grid(num_tiles, Hq, splits);
    pooled_attention_tile_kernel<kDimSteps, kValueTiles><<<grid, kTileThreads, smem, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (const __nv_bfloat16*)kp_cache,
        (const __nv_bfloat16*)vp_cache, block_table, table_width, pooled_table, pooled_width, cu, start_pos, tiles, v_table, v_rot,
        table_rows, (__nv_bfloat16*)out, Hq, Hkv, dim, vdim, page_size, scale, window, pool, splits > 1 ? partial : nullptr, splits,
        extras);
    return launch_status();
}

extern "C" int lb_pooled_attention_tile_q() { return kTileQ; }

// bfloat16 only; dim a multiple of 16 up to 128, vdim a multiple of 8 up to 128, an even v_rot.  With `splits` > 1 the chunks of
// every run are shared by that many CTAs and a merge over ALL `tokens` rows follows (`partial`: float32 scratch of tokens * Hq *
// splits * (vdim + 2); rows that no run covers hold whatever the scratch held: the caller writes them afterwards).
static int tile_dispatch(const void* q, const void* k_cache, const void* v_cache, const void* kp_cache,
                                        const void* vp_cache, const int* block_table, int table_width, const int* pooled_table,
                                        int pooled_width, const int* cu, const int* start_pos, const int* tiles, int num_tiles,
                                        const float* v_table, int v_rot, int table_rows, void* out, int Hq, int Hkv, int dim,
                                        int vdim, int page_size, float scale, int window, int pool, float* partial, int splits,
                                        ScoreExtras extras, void* stream) {
    if (num_tiles <= 0) return kOk;
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || Hq > 65535 || dim <= 0 || dim % 16 || vdim <= 0 || vdim % 8 || page_size <= 0 || window <= 0
        || pool < 0 || (v_rot & 1) || v_rot > vdim || table_rows <= 0)
        return kBadSize;
    if (dim > 128 || vdim > 128 || splits < 1 || splits > 64 || (splits > 1 && partial == nullptr)) return kTooLarge;
#define LB_TILE(DS, VT) return launch_tile<DS, VT>(q, k_cache, v_cache, kp_cache, vp_cache, block_table, table_width, pooled_table, \
        pooled_width, cu, start_pos, tiles, num_tiles, v_table, v_rot, table_rows, out, Hq, Hkv, dim, vdim, page_size, scale, window, pool, \
        partial, splits, extras, stream)
    const int ds = dim / 16, vt = vdim / 8;
    if (ds <= 2) { if (vt <= 4) LB_TILE(2, 4); if (vt <= 8) LB_TILE(2, 8); if (vt <= 12) LB_TILE(2, 12); LB_TILE(2, 16); }
    if (ds <= 4) { if (vt <= 4) LB_TILE(4, 4); if (vt <= 8) LB_TILE(4, 8); if (vt <= 12) LB_TILE(4, 12); LB_TILE(4, 16); }
    if (vt <= 4) LB_TILE(8, 4);
    if (vt <= 8) LB_TILE(8, 8);
    if (vt <= 12) LB_TILE(8, 12);
    LB_TILE(8, 16);
#undef LB_TILE
}

extern "C" int lb_pooled_attention_tile(const void* q, const void* k_cache, const void* v_cache, const void* kp_cache,
                                        const void* vp_cache, const int* block_table, int table_width, const int* pooled_table,
                                        int pooled_width, const int* cu, const int* start_pos, const int* tiles, int num_tiles,
                                        const int* positions, int tokens, const float* v_table, int v_rot, int table_rows, void* out,
                                        int Hq, int Hkv, int dim, int vdim, int page_size, float scale, int window, int pool,
                                        float* partial, int splits, const float* slopes, const float* sinks, void* stream) {
    // (with several CTAs per run the sink joins in the merge, once)
    const int code = tile_dispatch(q, k_cache, v_cache, kp_cache, vp_cache, block_table, table_width, pooled_table, pooled_width, cu,
                                   start_pos, tiles, num_tiles, v_table, v_rot, table_rows, out, Hq, Hkv, dim, vdim, page_size, scale,
                                   window, pool, partial, splits, ScoreExtras{slopes, splits > 1 ? nullptr : sinks}, stream);
    if (code != 0 || splits <= 1 || num_tiles <= 0 || tokens <= 0) return code;
    dim3 grid(tokens, Hq);
    pooled_merge_kernel<__nv_bfloat16><<<grid, 32, 0, (cudaStream_t)stream>>>(partial, positions, nullptr, v_table, v_rot, table_rows,
                                                                            (__nv_bfloat16*)out, Hq, vdim, splits, sinks);
    return launch_status();
}

// ------------------------------------------------------------------------------------------------------------------
// Queries and keys that are normed over the WHOLE projection (all heads of a token at once), then rotated; the values
// are the keys as they came in (before norm and rotation).
//
//   rownorm_prepare : per token, from qk = [q (Hq * dim) | k (Hkv * dim)]:
//                       q~ = q / sqrt(mean_all(q^2) + eps) * wq        (wq: a weight per column of the whole row)
//                       k~ = k / sqrt(mean_all(k^2) + eps) * wk
//                       q_out = R_p(q~),  k_cache[slot] = R_p(k~),  v_cache[slot] = k
//                     R_p turns neighbouring pairs (2i, 2i + 1) of the first `rot` columns of every head by the token's
//                     row of the table (cos | sin of rot / 2 pairs).  Norms and rotation are 32-bit.
//   head_gate       : o[t, h, :] *= sigmoid(g[t, h])                   (one gate per token and head, in place)
template <typename T>
__global__ void __launch_bounds__(256) rownorm_prepare_kernel(const T* __restrict__ qk, long row_stride, const int* __restrict__ positions,
                                                              const int* __restrict__ slot_mapping, const float* __restrict__ table, int rot,
                                                              int table_rows, const float* __restrict__ wq, const float* __restrict__ wk,
                                                              float eps, T* __restrict__ q_out, T* __restrict__ k_cache,
                                                              T* __restrict__ v_cache, int Hq, int Hkv, int dim, int write_kv) {
    __shared__ float red[32];
    const size_t t = blockIdx.x;
    const T* row = qk + t * row_stride;
    const int nq = Hq * dim, nk = Hkv * dim;
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) { const float v = to_f32(row[c]); sq += v * v; }
    for (int c = threadIdx.x; c < nk; c += blockDim.x) { const float v = to_f32(row[nq + c]); sk += v * v; }
    const float inv_q = 1.f / sqrtf(block_sum(sq, red) / (float)nq + eps);
    const float inv_k = 1.f / sqrtf(block_sum(sk, red) / (float)nk + eps);
    const int pos = min(max(positions[t], 0), table_rows - 1);
    const float* cs = table + (size_t)pos * rot;
    const int half = rot >> 1;
    const long slot = write_kv ? (long)slot_mapping[t] : -1;
    for (int c = threadIdx.x; c < nq + nk; c += blockDim.x) {
        const bool is_q = c < nq;
        const int cc = is_q ? c : c - nq;                    // column of the whole q (or k) row
        const int d = cc % dim;                              // column of its head
        const float* w = is_q ? wq : wk;
        const float inv = is_q ? inv_q : inv_k;
        const T* src = row + (is_q ? 0 : nq);
        const float raw = to_f32(src[cc]);
        float val = raw * inv * w[cc];
        if (d < rot) {
            const float partner = to_f32(src[cc ^ 1]) * inv * w[cc ^ 1];
            const float co = cs[d >> 1], si = cs[half + (d >> 1)];
            val = (d & 1) ? val * co + partner * si : val * co - partner * si;
        }
        if (is_q) q_out[t * nq + cc] = from_f32<T>(val);
        else if (slot >= 0) {
            k_cache[(size_t)slot * nk + cc] = from_f32<T>(val);
            v_cache[(size_t)slot * nk + cc] = src[cc];
        }
    }
}

// The same for bfloat16 rows whose columns come in aligned pairs (an even head size and row stride): a thread owns the pairs
// (2i, 2i + 1), which are also the rotation's pairs, and moves them as 4-byte words.
__global__ void __launch_bounds__(256) rownorm_prepare_pairs_kernel(const __nv_bfloat162* __restrict__ qk, long row_pairs,
                                                                    const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                                                                    const float* __restrict__ table, int rot, int table_rows,
                                                                    const float2* __restrict__ wq, const float2* __restrict__ wk, float eps,
                                                                    __nv_bfloat162* __restrict__ q_out, __nv_bfloat162* __restrict__ k_cache,
                                                                    __nv_bfloat162* __restrict__ v_cache, int Hq, int Hkv, int dim, int write_kv) {
    __shared__ float red[32];
    const size_t t = blockIdx.x;
    const __nv_bfloat162* row = qk + t * row_pairs;
    const int pq = Hq * dim / 2, pk = Hkv * dim / 2, pd = dim / 2;
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < pq; c += blockDim.x) { const float2 v = __bfloat1622float2(row[c]); sq += v.x * v.x + v.y * v.y; }
    for (int c = threadIdx.x; c < pk; c += blockDim.x) { const float2 v = __bfloat1622float2(row[pq + c]); sk += v.x * v.x + v.y * v.y; }
    const float inv_q = 1.f / sqrtf(block_sum(sq, red) / (float)(2 * pq) + eps);
    const float inv_k = 1.f / sqrtf(block_sum(sk, red) / (float)(2 * pk) + eps);
    const int pos = min(max(positions[t], 0), table_rows - 1);
    const float* cs = table + (size_t)pos * rot;
    const int half = rot >> 1;
    const long slot = write_kv ? (long)slot_mapping[t] : -1;
    for (int c = threadIdx.x; c < pq + pk; c += blockDim.x) {
        const bool is_q = c < pq;
        const int cc = is_q ? c : c - pq;
        const int d = cc % pd;                               // pair of its head
        const __nv_bfloat162 raw = row[c];
        const float2 v = __bfloat1622float2(raw), w = is_q ? wq[cc] : wk[cc];
        const float inv = is_q ? inv_q : inv_k;
        float a = v.x * inv * w.x, b = v.y * inv * w.y;
        if (d < half) {
            const float co = cs[d], si = cs[half + d];
            const float ra = a * co - b * si, rb = b * co + a * si;
            a = ra; b = rb;
        }
        const __nv_bfloat162 out = __floats2bfloat162_rn(a, b);
        if (is_q) q_out[t * pq + cc] = out;
        else if (slot >= 0) {
            k_cache[(size_t)slot * pk + cc] = out;
            v_cache[(size_t)slot * pk + cc] = raw;
        }
    }
}

// qk: [tokens, (Hq + Hkv) * dim] (column view allowed); table: float32 [table_rows, rot]; wq: float32 [Hq * dim];
// wk: float32 [Hkv * dim]; q_out: [tokens, Hq, dim]; caches: [slots, Hkv, dim], both
extern "C" int lb_rownorm_prepare(const void* qk, long row_stride, const int* positions, const int* slot_mapping, const float* table,
                                  int rot, int table_rows, const float* wq, const float* wk, float eps, void* q_out, void* k_cache,
                                  void* v_cache, int tokens, int Hq, int Hkv, int dim, int write_kv, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (Hq <= 0 || Hkv <= 0 || dim <= 0 || rot < 0 || rot > dim || (rot & 1) || table_rows <= 0) return kBadSize;
    if (dtype == kBF16 && dim % 2 == 0 && row_stride % 2 == 0 && ((uintptr_t)qk & 3) == 0 && ((uintptr_t)wq & 7) == 0 && ((uintptr_t)wk & 7) == 0) {
        typedef __nv_bfloat162 b2;
        rownorm_prepare_pairs_kernel<<<tokens, 256, 0, (cudaStream_t)stream>>>(
            (const b2*)qk, row_stride / 2, positions, slot_mapping, table, rot, table_rows, (const float2*)wq, (const float2*)wk, eps,
            (b2*)q_out, (b2*)k_cache, (b2*)v_cache, Hq, Hkv, dim, write_kv);
        return launch_status();
    }
    LB_DISPATCH_DTYPE(dtype, rownorm_prepare_kernel<T><<<tokens, 256, 0, (cudaStream_t)stream>>>(
        (const T*)qk, row_stride, positions, slot_mapping, table, rot, table_rows, wq, wk, eps, (T*)q_out, (T*)k_cache, (T*)v_cache,
        Hq, Hkv, dim, write_kv));
    return launch_status();
}

template <typename T, typename TG>
__global__ void head_gate_kernel(T* __restrict__ o, const TG* __restrict__ g, long g_stride, int H, int width, long total) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long t = i / ((long)H * width);
    const int h = (int)((i / width) % H);
    const float gate = 1.f / (1.f + expf(-to_f32(g[t * g_stride + h])));
    o[i] = from_f32<T>(to_f32(o[i]) * gate);
}

// bfloat16 rows of a width that is a multiple of 8: a thread scales 8 neighbouring columns of one head (one 16-byte word)
template <typename TG>
__global__ void head_gate_vec_kernel(uint4* __restrict__ o, const TG* __restrict__ g, long g_stride, int H, int groups, long total) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long th = i / groups;                             // (token, head)
    const long t = th / H;
    const int h = (int)(th % H);
    const float gate = 1.f / (1.f + expf(-to_f32(g[t * g_stride + h])));
    uint4 v = o[i];
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(p[e]); p[e] = __floats2bfloat162_rn(f.x * gate, f.y * gate); }
    o[i] = v;
}

// o: contiguous [tokens, H, width], scaled in place; g: [tokens, >= H] gate logits (float32 with `g_f32`, else o's dtype; row
// stride in elements)
extern "C" int lb_head_gate(void* o, const void* g, long g_stride, int g_f32, int tokens, int H, int width, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (H <= 0 || width <= 0) return kBadSize;
    const long total = (long)tokens * H * width;
    if (dtype == kBF16 && width % 8 == 0 && ((uintptr_t)o & 15) == 0) {
        const long words = total / 8;
        const unsigned vblocks = (unsigned)((words + 255) / 256);
        if (g_f32) head_gate_vec_kernel<float><<<vblocks, 256, 0, (cudaStream_t)stream>>>((uint4*)o, (const float*)g, g_stride, H, width / 8, words);
        else head_gate_vec_kernel<__nv_bfloat16><<<vblocks, 256, 0, (cudaStream_t)stream>>>((uint4*)o, (const __nv_bfloat16*)g, g_stride, H, width / 8, words);
        return launch_status();
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    LB_DISPATCH_DTYPE(dtype, {
        if (g_f32) head_gate_kernel<T, float><<<blocks, 256, 0, (cudaStream_t)stream>>>((T*)o, (const float*)g, g_stride, H, width, total);
        else head_gate_kernel<T, T><<<blocks, 256, 0, (cudaStream_t)stream>>>((T*)o, (const T*)g, g_stride, H, width, total);
    });
    return launch_status();
}
