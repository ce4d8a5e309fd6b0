// Routed feed-forward: the router, the experts' activation, identity experts, and the tanh GELU of dense layers.
//
//  moe_route        : 32-bit router per token: logits = W_r h, s = softmax over all n outputs (real and identity
//                     experts alike), or with `sigmoid_scores` s = sigmoid of each logit; the choice looks at
//                     s + correction (if there is one), restricted to the `keep` groups (of
//                     n / groups neighbours) whose best member scores highest; the `top` best are chosen; their
//                     weights are s * scale (no correction, no renormalisation).  With `sigmoid_scores` = 2 the
//                     logits themselves are ranked and the chosen ones' weights are the softmax over the chosen
//                     logits only (times scale).  `bias` (may be null) is added to the logits.  Writes the dense weights [T, n]
//                     (0 where not chosen), the chosen indices and weights [T, top], and per token the summed
//                     weight of the chosen identity experts (the last n - experts outputs).
//  moe_activation   : y[t, e, i] = w[t, e] * g~ * sigmoid(act_alpha * g~) * (u~ + 1),  g~ = min(g, limit),
//                     u~ = clamp(u, -limit, limit), from the packed [gate | up] products of all experts.  The expert's
//                     weight is applied here, so ONE product with the stacked down matrices sums the experts.
//                     Mode `kSiluInput`: y = silu(w g) * (w u), the expert silu(gate) * up on an input that was
//                     multiplied by the weight (gate and up are linear in it).  Without weights (`dense` null, one
//                     expert) it is the activation of a dense gated layer.  Modes `kSiluOutput` and `kGeluOutput`:
//                     y = w * silu(g) * u and y = w * gelu_tanh(g) * u.  Input and output rows may be column views
//                     of wider matrices (row strides in elements).
//  moe_add_identity : out += id_weight[t] * h
//  gelu_tanh        : 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
#include "lb200/common.cuh"
using namespace lb200;

constexpr int kRouteMax = 256;        // router outputs
constexpr int kRouteWarps = 16;       // warps of a token's CTA: each takes every sixteenth router output

// grid (tokens)
template <typename T>
__global__ void __launch_bounds__(kRouteWarps * 32) moe_route_kernel(
        const T* __restrict__ h, const float* __restrict__ w_router, const float* __restrict__ correction,
        float* __restrict__ dense, int* __restrict__ chosen, float* __restrict__ chosen_w,
        float* __restrict__ id_weight, int tokens, int width, int n, int experts, int top,
        int groups, int keep, float scale, int sigmoid_scores, const float* __restrict__ bias) {
    __shared__ float z[kRouteMax];
    __shared__ float c[kRouteMax];
    __shared__ unsigned char ok[kRouteMax];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x;
    const T* hr = h + (size_t)t * width;
    for (int e = warp; e < n; e += kRouteWarps) {
        const float* wr = w_router + (size_t)e * width;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        int k = lane;
#pragma unroll 2
        for (; k + 96 < width; k += 128) {
            a0 += to_f32(hr[k]) * wr[k];
            a1 += to_f32(hr[k + 32]) * wr[k + 32];
            a2 += to_f32(hr[k + 64]) * wr[k + 64];
            a3 += to_f32(hr[k + 96]) * wr[k + 96];
        }
        for (; k < width; k += 32) a0 += to_f32(hr[k]) * wr[k];
        const float a = warp_sum((a0 + a1) + (a2 + a3));
        if (lane == 0) z[e] = a + (bias != nullptr ? bias[e] : 0.f);
    }
    __syncthreads();
    if (warp != 0) return;
    const bool chosen_softmax = sigmoid_scores == 2;
    float mx = 0.f, sum = 1.f;
    if (sigmoid_scores == 0) {
        mx = -INFINITY;
        for (int e = lane; e < n; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        sum = 0.f;
        for (int e = lane; e < n; e += 32) sum += expf(z[e] - mx);
        sum = warp_sum(sum);
    }
    __syncwarp();
    for (int e = lane; e < n; e += 32) {
        const float logit = z[e];
        const float s = chosen_softmax ? logit : (sigmoid_scores ? 1.f / (1.f + expf(-logit)) : expf(logit - mx) / sum);
        z[e] = s;
        // sigmoid scores without a correction are ranked by their logits: the same order, and two large logits do not
        // meet in a score that has rounded to 1
        c[e] = (sigmoid_scores && correction == nullptr) ? logit : s + (correction != nullptr ? correction[e] : 0.f);
        ok[e] = 0;
        dense[(size_t)t * n + e] = 0.f;
    }
    __syncwarp();
    if (lane != 0) return;
    // the groups that stay: `keep` times the group whose best member is largest (ties: the lower index)
    const int per = n / groups;
    for (int r = 0; r < keep; ++r) {
        int best_g = -1;
        float best = -INFINITY;
        for (int g = 0; g < groups; ++g) {
            if (ok[g * per]) continue;
            float gm = -INFINITY;
            for (int i = 0; i < per; ++i) gm = fmaxf(gm, c[g * per + i]);
            if (best_g < 0 || gm > best) { best = gm; best_g = g; }
        }
        if (best_g < 0) break;
        for (int i = 0; i < per; ++i) ok[best_g * per + i] = 1;
    }
    float idw = 0.f;
    if (chosen_softmax) {
        // the `top` largest logits, then the softmax over them alone
        float best_all = -INFINITY, total = 0.f;
        for (int r = 0; r < top; ++r) {
            int best_e = -1;
            float best = -INFINITY;
            for (int e = 0; e < n; ++e)
                if (ok[e] == 1 && (best_e < 0 || c[e] > best)) { best = c[e]; best_e = e; }
            chosen[(size_t)t * top + r] = best_e;
            if (best_e < 0) { chosen_w[(size_t)t * top + r] = 0.f; continue; }
            ok[best_e] = 2;
            if (r == 0) best_all = best;
            const float p = expf(best - best_all);
            chosen_w[(size_t)t * top + r] = p;
            total += p;
        }
        for (int r = 0; r < top; ++r) {
            const int e = chosen[(size_t)t * top + r];
            if (e < 0) continue;
            const float wgt = chosen_w[(size_t)t * top + r] / total * scale;
            chosen_w[(size_t)t * top + r] = wgt;
            dense[(size_t)t * n + e] = wgt;
            if (e >= experts) idw += wgt;
        }
        id_weight[t] = idw;
        return;
    }
    for (int r = 0; r < top; ++r) {
        int best_e = -1;
        float best = -INFINITY;
        for (int e = 0; e < n; ++e)
            if (ok[e] == 1 && (best_e < 0 || c[e] > best)) { best = c[e]; best_e = e; }
        if (best_e < 0) { chosen[(size_t)t * top + r] = -1; chosen_w[(size_t)t * top + r] = 0.f; continue; }
        ok[best_e] = 2;
        const float wgt = z[best_e] * scale;
        dense[(size_t)t * n + best_e] = wgt;
        chosen[(size_t)t * top + r] = best_e;
        chosen_w[(size_t)t * top + r] = wgt;
        if (best_e >= experts) idw += wgt;
    }
    id_weight[t] = idw;
}

extern "C" int lb_moe_route(const void* h, const float* w_router, const float* correction, float* dense, int* chosen,
                            float* chosen_w, float* id_weight, int tokens, int width, int n, int experts, int top, int groups,
                            int keep, float scale, int sigmoid_scores, const float* bias, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (n <= 0 || experts < 0 || experts > n || top <= 0 || top > n || groups <= 0 || n % groups || keep <= 0 || keep > groups)
        return kBadSize;
    if (n > kRouteMax) return kTooLarge;
    if (sigmoid_scores < 0 || sigmoid_scores > 2) return kBadSize;
    LB_DISPATCH_DTYPE(dtype, moe_route_kernel<T><<<tokens, kRouteWarps * 32, 0, (cudaStream_t)stream>>>(
        (const T*)h, w_router, correction, dense, chosen, chosen_w, id_weight, tokens, width, n, experts, top, groups, keep, scale, sigmoid_scores, bias));
    return launch_status();
}

enum : int { kClampedOutput = 0, kSiluInput = 1, kSiluOutput = 2, kGeluOutput = 3 };

__device__ __forceinline__ float gelu_tanh_f(float z) { return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

__device__ __forceinline__ float expert_act(float g, float u, float w, float limit, float act_alpha, int mode) {
    if (mode == kSiluInput) {
        const float wg = w * g;
        return wg / (1.f + expf(-wg)) * (w * u);
    }
    if (mode == kSiluOutput) return w * (g / (1.f + expf(-g)) * u);
    if (mode == kGeluOutput) return w * (gelu_tanh_f(g) * u);
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return w * (g / (1.f + expf(-act_alpha * g)) * (u + 1.f));
}

// gu: [T, experts, 2, ff]; y: [T, experts, ff]; dense: [T, n] (null: weight 1)
template <typename T>
__global__ void moe_activation_kernel(const T* __restrict__ gu, const float* __restrict__ dense, T* __restrict__ y,
                                      int experts, int ff, int n, float limit, float act_alpha, int mode, long in_stride,
                                      long out_stride) {
    const size_t t = blockIdx.z;
    const int e = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= ff) return;
    const float w = dense != nullptr ? dense[t * n + e] : 1.f;
    float v = 0.f;
    if (w != 0.f) {
        const T* row = gu + t * in_stride + e * 2 * (size_t)ff;
        v = expert_act(to_f32(row[i]), to_f32(row[ff + i]), w, limit, act_alpha, mode);
    }
    y[t * out_stride + e * (size_t)ff + i] = from_f32<T>(v);
}

// the same for bfloat16 rows with ff a multiple of 8: a CTA per token walks its experts' rows in 16-byte pieces, and writes
// zeros for the experts that were not chosen without reading their products
__global__ void __launch_bounds__(256) moe_activation_vec_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ dense,
                                                                 __nv_bfloat16* __restrict__ y, int experts, int ff, int n,
                                                                 float limit, float act_alpha, int mode, long in_stride,
                                                                 long out_stride) {
    const size_t t = blockIdx.x;
    const int pieces = ff / 8;
    for (int i = threadIdx.x; i < experts * pieces; i += blockDim.x) {
        const int e = i / pieces, pc = i % pieces;
        const float w = dense != nullptr ? dense[t * n + e] : 1.f;
        uint4 out = make_uint4(0, 0, 0, 0);
        if (w != 0.f) {
            const __nv_bfloat16* row = gu + t * in_stride + e * 2 * (size_t)ff;
            const uint4 gv = *reinterpret_cast<const uint4*>(row + pc * 8);
            const uint4 uv = *reinterpret_cast<const uint4*>(row + ff + pc * 8);
            const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
            const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
                if (mode == kSiluInput) {
                    const float g0 = w * g.x, g1 = w * g.y;
                    o2[k] = __floats2bfloat162_rn(__fdividef(g0, 1.f + __expf(-g0)) * (w * u.x), __fdividef(g1, 1.f + __expf(-g1)) * (w * u.y));
                } else if (mode == kSiluOutput) {
                    o2[k] = __floats2bfloat162_rn(w * (__fdividef(g.x, 1.f + __expf(-g.x)) * u.x), w * (__fdividef(g.y, 1.f + __expf(-g.y)) * u.y));
                } else if (mode == kGeluOutput) {
                    o2[k] = __floats2bfloat162_rn(w * (gelu_tanh_f(g.x) * u.x), w * (gelu_tanh_f(g.y) * u.y));
                } else {
                    const float g0 = fminf(g.x, limit), g1 = fminf(g.y, limit);
                    const float u0 = fminf(fmaxf(u.x, -limit), limit), u1 = fminf(fmaxf(u.y, -limit), limit);
                    o2[k] = __floats2bfloat162_rn(w * (g0 / (1.f + __expf(-act_alpha * g0)) * (u0 + 1.f)),
                                                  w * (g1 / (1.f + __expf(-act_alpha * g1)) * (u1 + 1.f)));
                }
            }
        }
        *reinterpret_cast<uint4*>(y + t * out_stride + e * (size_t)ff + pc * 8) = out;
    }
}

extern "C" int lb_moe_activation(const void* gu, const float* dense, void* y, int tokens, int experts, int ff, int n, float limit,
                                 float act_alpha, int mode, long in_stride, long out_stride, int dtype, void* stream) {
    if (tokens <= 0 || experts <= 0) return kOk;
    if (ff <= 0 || (dense != nullptr && n < experts) || experts > 65535 || mode < kClampedOutput || mode > kGeluOutput
        || in_stride < 2 * (long)experts * ff || out_stride < (long)experts * ff)
        return kBadSize;
    if (dtype == kBF16 && ff % 8 == 0 && (((uintptr_t)gu | (uintptr_t)y) & 15) == 0 && in_stride % 8 == 0 && out_stride % 8 == 0) {
        moe_activation_vec_kernel<<<tokens, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu, dense, (__nv_bfloat16*)y, experts, ff,
                                                                          n, limit, act_alpha, mode, in_stride, out_stride);
        return launch_status();
    }
    dim3 grid((ff + 127) / 128, experts, tokens);
    LB_DISPATCH_DTYPE(dtype, moe_activation_kernel<T><<<grid, 128, 0, (cudaStream_t)stream>>>(
        (const T*)gu, dense, (T*)y, experts, ff, n, limit, act_alpha, mode, in_stride, out_stride));
    return launch_status();
}

template <typename T>
__global__ void moe_add_identity_kernel(T* __restrict__ out, const T* __restrict__ h, const float* __restrict__ id_weight, int width) {
    const size_t t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const float w = id_weight[t];
    if (w != 0.f) out[t * width + c] = from_f32<T>(to_f32(out[t * width + c]) + w * to_f32(h[t * width + c]));
}

extern "C" int lb_moe_add_identity(void* out, const void* h, const float* id_weight, int tokens, int width, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (width <= 0) return kBadSize;
    dim3 grid((width + 255) / 256, tokens);
    LB_DISPATCH_DTYPE(dtype, moe_add_identity_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>((T*)out, (const T*)h, id_weight, width));
    return launch_status();
}

template <typename T>
__global__ void gelu_tanh_kernel(const T* __restrict__ in, T* __restrict__ out, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float z = to_f32(in[i]);
    out[i] = from_f32<T>(0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))));
}

extern "C" int lb_gelu_tanh(const void* in, void* out, long n, int dtype, void* stream) {
    if (n <= 0) return kOk;
    LB_DISPATCH_DTYPE(dtype, gelu_tanh_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const T*)in, (T*)out, (size_t)n));
    return launch_status();
}

// x[t, c] <- silu(x[t, c] * scale[c]) for the first `cols` columns of every row (row stride in elements; scale may be null)
template <typename T>
__global__ void silu_columns_kernel(T* __restrict__ x, long stride, int cols, const float* __restrict__ scale, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int c = (int)(i % cols);
    T* at = x + (i / cols) * stride + c;
    float v = to_f32(*at);
    if (scale != nullptr) v = round_to<T>(v * scale[c]);
    *at = from_f32<T>(silu_f(v));
}

extern "C" int lb_silu_columns(void* x, long stride, int rows, int cols, const float* scale, int dtype, void* stream) {
    if (rows <= 0 || cols <= 0) return kOk;
    if (stride < cols) return kBadSize;
    const size_t total = (size_t)rows * cols;
    LB_DISPATCH_DTYPE(dtype, silu_columns_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((T*)x, stride, cols, scale, total));
    return launch_status();
}
