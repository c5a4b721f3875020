// Routed feed-forward (mixture of experts): the router, and the experts for few rows.
//
// Router, per row x (float arithmetic throughout):
//   z = W_r x,  s = softmax(z) over all experts (identity experts included), or s = sigmoid(z) expert by expert,
//   choice = s + correction;  the `top` largest choices are taken (ties: the lower index),
//   their weights are s itself (not renormalised).
//   A third scoring: z = W_r x + b, the `top` largest z are taken and their weights are the softmax over those z alone.
// An expert e < n_real is a gated feed-forward, y = W_down act(W_gate x, W_up x); an expert e >= n_real is
// an identity expert whose output is x.  The row's result is sum_k weight_k y_k in the order of the choice.
// Two further forms: experts of two matrices, y = W_down act(W_up x) (activation codes RDL_UNARY_*), and weights
// that multiply an expert's input instead of its output, y_k = expert(weight_k x), summed with weight one.
//
// Few rows (single-token steps, the 32-bit path): every (row, choice) pair streams its expert's
// matrices, a warp per output value (rdl_moe_gate_up, rdl_moe_down_combine); the sums run lane by lane
// over k in an order that depends on k alone.  Many rows are sorted by expert and go through the tiled
// product with one expert per row tile (rdl_moe_align, rdl_moe_gather, rdl_gemm_tc_grouped, rdl_moe_combine).
#include "activations.cuh"
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

// Router logits z[t, e] = W_r[e, :] . x[t, :] in float, two forms; in both a (row, expert) sum is formed in an order
// that depends on the width alone.
//   many rows: a block takes 16 rows and 8 experts, a warp one expert for all of the block's rows (a weight row is
//     read once for them), lanes split k;
//   few rows (single-token steps): a block takes one expert and up to 8 rows, its 8 warps split k, so that every load of
//     the sum is in flight at once; the warps' parts are added in a fixed order through shared memory.
constexpr int ROUTE_WARPS = 8, ROUTE_FEW_ROWS = 8, ROUTE_MANY_ROWS = 16, ROUTE_CHUNK = 256;

// four consecutive values as floats (8- or 16-byte load)
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }

template <typename T, int ROWS, bool SPLIT_K>
__global__ void __launch_bounds__(ROUTE_WARPS * 32) moe_logits_kernel(const T* __restrict__ x, const float* __restrict__ w_router, int n_rows,
                                                                      int n_experts, int width, float* __restrict__ z) {
    __shared__ float part[ROUTE_WARPS][ROWS];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * ROWS;
    const int e = SPLIT_K ? blockIdx.y : blockIdx.y * ROUTE_WARPS + warp;
    const bool live = e < n_experts;
    const int rows = min(ROWS, n_rows - t0);
    const float* w = w_router + (long long)(live ? e : 0) * width;
    float acc[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
    // SPLIT_K: all threads of the block walk k together; else a warp walks k alone
    const int first = SPLIT_K ? threadIdx.x : lane, stride = SPLIT_K ? ROUTE_WARPS * 32 : 32;
    const bool pieces = width % 4 == 0 && ((uintptr_t)w_router & 15) == 0 && ((uintptr_t)x & 15) == 0;
    if (!SPLIT_K && pieces) {
        // The block's rows pass through shared memory, 256 values of each at a time, as floats: its eight warps read the
        // same rows, and what one warp brought in would not wait in L1 for the others.  A lane still meets k in the order
        // lane * 4 + {0, 128, 256, ...}.
        __shared__ __align__(16) float xs[SPLIT_K ? 1 : ROWS][ROUTE_CHUNK];
        for (int k0 = 0; k0 < width; k0 += ROUTE_CHUNK) {
            for (int idx = threadIdx.x; idx < ROWS * (ROUTE_CHUNK / 4); idx += ROUTE_WARPS * 32) {
                const int r = idx / (ROUTE_CHUNK / 4), kk = (idx - r * (ROUTE_CHUNK / 4)) * 4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (r < rows && k0 + kk < width) v = load4(x + (long long)(t0 + r) * width + k0 + kk);
                *reinterpret_cast<float4*>(&xs[r][kk]) = v;
            }
            __syncthreads();
            if (live) {
                for (int kk = lane * 4; kk < ROUTE_CHUNK && k0 + kk < width; kk += 128) {
                    const float4 wv = *reinterpret_cast<const float4*>(w + k0 + kk);
#pragma unroll
                    for (int r = 0; r < ROWS; ++r) {
                        const float4 xv = *reinterpret_cast<const float4*>(&xs[r][kk]);
                        acc[r] = fmaf(wv.x, xv.x, acc[r]);
                        acc[r] = fmaf(wv.y, xv.y, acc[r]);
                        acc[r] = fmaf(wv.z, xv.z, acc[r]);
                        acc[r] = fmaf(wv.w, xv.w, acc[r]);
                    }
                }
            }
            __syncthreads();
        }
    } else if (live) {
        if (pieces) {
            for (int k = first * 4; k < width; k += stride * 4) {
                const float4 wv = *reinterpret_cast<const float4*>(w + k);
                float4 xv[ROWS];                           // every row's piece is asked for before any is used
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    xv[r] = r < rows ? load4(x + (long long)(t0 + r) * width + k) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    acc[r] = fmaf(wv.x, xv[r].x, acc[r]);
                    acc[r] = fmaf(wv.y, xv[r].y, acc[r]);
                    acc[r] = fmaf(wv.z, xv[r].z, acc[r]);
                    acc[r] = fmaf(wv.w, xv[r].w, acc[r]);
                }
            }
        } else {
            for (int k = first; k < width; k += stride) {
                const float wv = w[k];
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    if (r < rows) acc[r] = fmaf(wv, to_float(x[(long long)(t0 + r) * width + k]), acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = warp_sum(acc[r]);
    if (!SPLIT_K) {
        if (live && lane == 0) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (r < rows) z[(long long)(t0 + r) * n_experts + e] = acc[r];
        }
        return;
    }
    if (lane == 0)
#pragma unroll
        for (int r = 0; r < ROWS; ++r) part[warp][r] = acc[r];
    __syncthreads();
    if (threadIdx.x < rows) {
        float v = 0.f;
#pragma unroll
        for (int wdx = 0; wdx < ROUTE_WARPS; ++wdx) v += part[wdx][threadIdx.x];
        z[(long long)(t0 + threadIdx.x) * n_experts + e] = v;
    }
}

// softmax over a row's logits, choice = score + correction, the `top` largest choices: a warp per row
constexpr int TOPK_WARPS = 4;

__global__ void __launch_bounds__(TOPK_WARPS * 32) moe_topk_kernel(const float* __restrict__ z, const float* __restrict__ bias,
                                                                   const float* __restrict__ correction, int n_rows,
                                                                   int n_experts, int top, int scoring, int* __restrict__ sel,
                                                                   float* __restrict__ sel_w) {
    extern __shared__ float zs_all[];          // per warp: [n_experts] scores, [n_experts] choices, [top] chosen scores
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * TOPK_WARPS + warp;
    if (t >= n_rows) return;
    float* zs = zs_all + (size_t)warp * (2 * n_experts + top);
    float* choice = zs + n_experts;
    float* picked = choice + n_experts;
    const float* zr = z + (long long)t * n_experts;
    float m = -INFINITY;
    float sum = 1.f;
    auto logit = [&](int e) { return bias ? zr[e] + bias[e] : zr[e]; };
    if (scoring == RDL_ROUTE_SOFTMAX_CHOSEN) {
        for (int e = lane; e < n_experts; e += 32) zs[e] = logit(e);
    } else if (scoring == RDL_ROUTE_SIGMOID) {
        for (int e = lane; e < n_experts; e += 32) zs[e] = 1.0f / (1.0f + expf(-logit(e)));
    } else {
        for (int e = lane; e < n_experts; e += 32) m = fmaxf(m, logit(e));
        m = warp_max(m);
        sum = 0.f;
        for (int e = lane; e < n_experts; e += 32) {
            const float p = expf(logit(e) - m);
            zs[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
    }
    __syncwarp();
    for (int e = lane; e < n_experts; e += 32) {
        const float s = scoring == RDL_ROUTE_SOFTMAX ? zs[e] / sum : zs[e];
        zs[e] = s;
        choice[e] = s + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float c = choice[e];
            if (c > best) { best = c; best_e = e; }       // lanes see their experts in rising order: the lower index wins a tie
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e == 0x7fffffff) best_e = 0;              // only if every remaining choice is NaN or -inf
        if (lane == 0) {
            sel[(long long)t * top + k] = best_e;
            if (scoring == RDL_ROUTE_SOFTMAX_CHOSEN) picked[k] = zs[best_e];
            else sel_w[(long long)t * top + k] = zs[best_e];
            choice[best_e] = -INFINITY;
        }
        __syncwarp();
    }
    if (scoring == RDL_ROUTE_SOFTMAX_CHOSEN && lane == 0) {
        // the weights: a softmax over the chosen logits alone (the first chosen is the largest), summed in the order of the choice
        const float top_logit = picked[0];
        float total = 0.f;
        for (int k = 0; k < top; ++k) { picked[k] = expf(picked[k] - top_logit); total += picked[k]; }
        for (int k = 0; k < top; ++k) sel_w[(long long)t * top + k] = picked[k] / total;
    }
}

constexpr int PAIR_WARPS = 8;

// A lane's share of sum_i a[i] * b[i] (and of a second row a2 with the same b): 16-byte loads where n and the
// addresses allow (bfloat16: 8 values, float: 4), else value by value.  Which form runs depends on n and on where
// rows start, never on the step's row count.
template <typename T> struct Piece;
template <> struct Piece<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(h[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
    }
};
template <> struct Piece<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
};
template <typename T>
__device__ __forceinline__ bool pieces_ok(const T* a, const T* b, int n) {
    return n % Piece<T>::N == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0;
}
template <typename T>
__device__ __forceinline__ void lane_dot2(const T* a1, const T* a2, const T* b, int n, int lane, float& s1, float& s2) {
    constexpr int N = Piece<T>::N;
    s1 = 0.f; s2 = 0.f;
    if (pieces_ok(a1, b, n) && (((uintptr_t)a2) & 15) == 0) {
        for (int i = lane * N; i < n; i += 32 * N) {
            float x[N], w1[N], w2[N];
            Piece<T>::load(b + i, x);
            Piece<T>::load(a1 + i, w1);
            Piece<T>::load(a2 + i, w2);
#pragma unroll
            for (int j = 0; j < N; ++j) { s1 = fmaf(w1[j], x[j], s1); s2 = fmaf(w2[j], x[j], s2); }
        }
    } else {
        for (int i = lane; i < n; i += 32) {
            const float x = to_float(b[i]);
            s1 = fmaf(to_float(a1[i]), x, s1);
            s2 = fmaf(to_float(a2[i]), x, s2);
        }
    }
}
template <typename T>
__device__ __forceinline__ float lane_dot(const T* a, const T* b, int n, int lane) {
    constexpr int N = Piece<T>::N;
    float s = 0.f;
    if (pieces_ok(a, b, n)) {
        for (int i = lane * N; i < n; i += 32 * N) {
            float x[N], w[N];
            Piece<T>::load(b + i, x);
            Piece<T>::load(a + i, w);
#pragma unroll
            for (int j = 0; j < N; ++j) s = fmaf(w[j], x[j], s);
        }
    } else {
        for (int i = lane; i < n; i += 32) s = fmaf(to_float(a[i]), to_float(b[i]), s);
    }
    return s;
}

// mid[p, j] = act(W_gate[e] x, W_up[e] x)[j] for pair p = (row t, choice k) with expert e = sel[p] < n_real.
// w: [n_real][2 ff][width], an expert's gate rows followed by its up rows.  A warp per (pair, j).
// activation >= 16: experts of two matrices, w [n_real][ff][width], mid = act(W_up[e] x).  sel_w given: the pair's weight
// multiplies the expert's input; a product is linear in it, so it multiplies the float sums instead of every term.
template <typename T>
__global__ void __launch_bounds__(PAIR_WARPS * 32) moe_gate_up_kernel(T* __restrict__ mid, const T* __restrict__ x, const T* __restrict__ w,
                                                                      const int* __restrict__ sel, const float* __restrict__ sel_w, int top,
                                                                      int n_real, int ff, int width, int activation, float act_param) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int p = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = sel[p];
    if (e < 0 || e >= n_real) return;
    const int j = blockIdx.x * PAIR_WARPS + warp;
    if (j >= ff) return;
    const T* row = x + (long long)(p / top) * width;
    const float in_w = sel_w ? sel_w[p] : 1.0f;
    if (activation >= 16) {
        const float u = warp_sum(lane_dot<T>(w + ((long long)e * ff + j) * width, row, width, lane)) * in_w;
        const float r = fmaxf(u, 0.f);
        if (lane == 0) mid[(long long)p * ff + j] = from_float<T>(activation == RDL_UNARY_RELU2 ? r * r : u / (1.0f + expf(-u)));
        return;
    }
    const T* wg = w + ((long long)e * 2 * ff + j) * width;
    const T* wu = wg + (long long)ff * width;
    float g, u;
    lane_dot2<T>(wg, wu, row, width, lane, g, u);
    g = warp_sum(g) * in_w;
    u = warp_sum(u) * in_w;
    if (lane == 0) mid[(long long)p * ff + j] = from_float<T>(rdl_gated(g, u, activation, act_param));
}

// out[t, n] = sum_k sel_w[t, k] * (expert k real ? W_down[e_k][n, :] . mid[(t, k), :] : x[t, n]), k in rising order.
template <typename T>
__global__ void __launch_bounds__(PAIR_WARPS * 32) moe_down_combine_kernel(T* __restrict__ out, const T* __restrict__ mid, const T* __restrict__ x,
                                                                           const T* __restrict__ w_down, const int* __restrict__ sel,
                                                                           const float* __restrict__ sel_w, int top, int n_real, int ff,
                                                                           int width) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * PAIR_WARPS + warp;
    if (n >= width) return;
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        const int p = t * top + k;
        const int e = sel[p];
        const float wk = sel_w ? sel_w[p] : 1.0f;
        float y;
        if (e >= n_real) {
            y = to_float(x[(long long)t * width + n]);
        } else {
            const T* w = w_down + ((long long)e * width + n) * ff;
            const T* m = mid + (long long)p * ff;
            y = warp_sum(lane_dot<T>(w, m, ff, lane));
        }
        total = fmaf(wk, y, total);
    }
    if (lane == 0) out[(long long)t * width + n] = from_float<T>(total);
}

// ---- many rows: sorted by expert, one expert per tile of MOE_TILE rows ----

constexpr int MOE_TILE = 128, ALIGN_THREADS = 1024;

// Gives every (row, choice) pair with a real expert a slot in a buffer in which each expert's pairs lie together,
// every expert's run padded to whole tiles: pair_slot[p] (-1: an identity expert), slot_pair[s] (-1: padding),
// tile_group[tile] (the tile's expert; -1: not in use).  One block; shared memory: 3 n_real + 1 ints.
__global__ void __launch_bounds__(ALIGN_THREADS) moe_align_kernel(const int* __restrict__ sel, int n_pairs, int n_real, int max_tiles,
                                                                  int* __restrict__ pair_slot, int* __restrict__ slot_pair,
                                                                  int* __restrict__ tile_group) {
    extern __shared__ int ws[];
    int* counts = ws;
    int* offsets = ws + n_real;            // n_real + 1 entries
    int* cursor = ws + 2 * n_real + 1;
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    for (int e = threadIdx.x; e < n_real; e += ALIGN_THREADS) { counts[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += ALIGN_THREADS) {
        const int e = sel[p];
        if (e >= 0 && e < n_real) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0;
        for (int e = 0; e < n_real; ++e) {
            offsets[e] = off;
            off += (counts[e] + MOE_TILE - 1) / MOE_TILE * MOE_TILE;
        }
        offsets[n_real] = off;
    }
    __syncthreads();
    for (int t = threadIdx.x; t < max_tiles; t += ALIGN_THREADS) {
        const int row = t * MOE_TILE;
        int g = -1;
        if (row < offsets[n_real]) {
            int lo = 0, hi = n_real - 1;   // the last expert whose run starts at or before the row (empty runs start where the next one does)
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (offsets[mid] <= row) lo = mid; else hi = mid - 1;
            }
            g = lo;
        }
        tile_group[t] = g;
    }
    for (int s = threadIdx.x; s < max_tiles * MOE_TILE; s += ALIGN_THREADS) slot_pair[s] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += ALIGN_THREADS) {
        const int e = sel[p];
        int slot = -1;
        if (e >= 0 && e < n_real) {
            slot = offsets[e] + atomicAdd(&cursor[e], 1);
            slot_pair[slot] = p;
        }
        pair_slot[p] = slot;
    }
}

// xs[slot, :] = x[pair / top, :] (zeros in padding slots of tiles in use); 16-byte pieces
__global__ void moe_gather_kernel(uint4* __restrict__ xs, const uint4* __restrict__ x, const int* __restrict__ slot_pair,
                                  const int* __restrict__ tile_group, const float* __restrict__ sel_w, int top, int pieces) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int slot = blockIdx.x;
    if (tile_group[slot / MOE_TILE] < 0) return;
    const int p = slot_pair[slot];
    uint4* dst = xs + (long long)slot * pieces;
    if (p < 0) {
        for (int i = threadIdx.x; i < pieces; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    } else {
        const uint4* src = x + (long long)(p / top) * pieces;
        if (!sel_w) {
            for (int i = threadIdx.x; i < pieces; i += blockDim.x) dst[i] = src[i];
        } else {
            const float wk = sel_w[p];
            for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
                uint4 raw = src[i];
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 v = __bfloat1622float2(h[k]);
                    h[k] = __floats2bfloat162_rn(v.x * wk, v.y * wk);
                }
                dst[i] = raw;
            }
        }
    }
}

// out[t, :] = sum_k sel_w[t, k] * (pair_slot[(t, k)] >= 0 ? y[slot, :] : x[t, :]), k in rising order, float sums
__global__ void moe_combine_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x,
                                   const int* __restrict__ pair_slot, const float* __restrict__ sel_w, int top, int width) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x;
    for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        for (int k = 0; k < top; ++k) {
            const int slot = pair_slot[t * top + k];
            const float wk = sel_w ? sel_w[t * top + k] : 1.0f;
            const __nv_bfloat16* src = slot >= 0 ? y + (long long)slot * width + c : x + (long long)t * width + c;
            const uint4 raw = *reinterpret_cast<const uint4*>(src);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 v = __bfloat1622float2(h[i]);
                acc[2 * i] = fmaf(wk, v.x, acc[2 * i]);
                acc[2 * i + 1] = fmaf(wk, v.y, acc[2 * i + 1]);
            }
        }
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        *reinterpret_cast<uint4*>(out + (long long)t * width + c) = raw;
    }
}

}  // namespace

extern "C" int rdl_moe_route(const void* x, int dtype, const float* w_router, const float* bias, const float* correction, int n_rows,
                             int n_experts, int width, int top, int scoring, int* sel, float* sel_w, float* logits, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "moe_route: bad dtype %d", dtype);
    RDL_REQUIRE(x && w_router && sel && sel_w && logits && n_experts > 0 && width > 0, "moe_route: bad arguments");
    RDL_REQUIRE(top >= 1 && top <= n_experts, "moe_route: %d of %d experts cannot be chosen", top, n_experts);
    RDL_REQUIRE(scoring == RDL_ROUTE_SOFTMAX || scoring == RDL_ROUTE_SIGMOID || scoring == RDL_ROUTE_SOFTMAX_CHOSEN, "moe_route: unknown scoring %d", scoring);
    RDL_REQUIRE(n_experts <= 1024, "moe_route: %d experts exceed the 1,024 the router kernels hold", n_experts);
    if (n_rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    // few rows: a block per expert with k split between its warps; many rows: 16 rows and 8 experts a block
    // (the two forms add a row's terms up in different orders: the 32-bit path, whose results must not depend on a step's
    // row count, always takes the first)
    const bool few = n_rows <= 64 || dtype == RDL_F32;
    const dim3 block(ROUTE_WARPS * 32);
    const dim3 grid = few ? dim3((n_rows + ROUTE_FEW_ROWS - 1) / ROUTE_FEW_ROWS, n_experts)
                          : dim3((n_rows + ROUTE_MANY_ROWS - 1) / ROUTE_MANY_ROWS, (n_experts + ROUTE_WARPS - 1) / ROUTE_WARPS);
    if (dtype == RDL_BF16) {
        const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
        if (few) RDL_CHECK_EX(rdl_launch(moe_logits_kernel<__nv_bfloat16, ROUTE_FEW_ROWS, true>, grid, block, 0, st, xp, w_router, n_rows, n_experts, width, logits), "moe_route");
        else RDL_CHECK_EX(rdl_launch(moe_logits_kernel<__nv_bfloat16, ROUTE_MANY_ROWS, false>, grid, block, 0, st, xp, w_router, n_rows, n_experts, width, logits), "moe_route");
    } else {
        const float* xp = (const float*)x;
        if (few) RDL_CHECK_EX(rdl_launch(moe_logits_kernel<float, ROUTE_FEW_ROWS, true>, grid, block, 0, st, xp, w_router, n_rows, n_experts, width, logits), "moe_route");
        else RDL_CHECK_EX(rdl_launch(moe_logits_kernel<float, ROUTE_MANY_ROWS, false>, grid, block, 0, st, xp, w_router, n_rows, n_experts, width, logits), "moe_route");
    }
    const size_t smem = (size_t)TOPK_WARPS * (2 * n_experts + top) * sizeof(float);
    RDL_CHECK_EX(rdl_launch(moe_topk_kernel, dim3((n_rows + TOPK_WARPS - 1) / TOPK_WARPS), dim3(TOPK_WARPS * 32), smem, st, (const float*)logits,
                            bias, correction, n_rows, n_experts, top, scoring, sel, sel_w), "moe_route");
    return 0;
}

extern "C" int rdl_moe_gate_up(void* mid, int dtype, const void* x, const void* w_gate_up, const int* sel, const float* sel_w, int n_rows,
                               int top, int n_real, int ff, int width, int activation, float act_param, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "moe_gate_up: bad dtype %d", dtype);
    RDL_REQUIRE(mid && x && sel && (w_gate_up || n_real == 0) && top > 0 && ff > 0 && width > 0, "moe_gate_up: bad arguments");
    RDL_REQUIRE(rdl_gated_known(activation) || activation == RDL_UNARY_RELU2 || activation == RDL_UNARY_SILU,
                "moe_gate_up: unknown activation %d", activation);
    if (n_rows == 0 || n_real == 0) return 0;
    RDL_REQUIRE((long long)n_rows * top <= 65535, "moe_gate_up: %d rows x %d choices exceed the grid limit", n_rows, top);
    const dim3 grid((ff + PAIR_WARPS - 1) / PAIR_WARPS, n_rows * top);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == RDL_BF16)
        RDL_CHECK_EX(rdl_launch(moe_gate_up_kernel<__nv_bfloat16>, grid, dim3(PAIR_WARPS * 32), 0, st, (__nv_bfloat16*)mid, (const __nv_bfloat16*)x,
                                (const __nv_bfloat16*)w_gate_up, sel, sel_w, top, n_real, ff, width, activation, act_param), "moe_gate_up");
    else
        RDL_CHECK_EX(rdl_launch(moe_gate_up_kernel<float>, grid, dim3(PAIR_WARPS * 32), 0, st, (float*)mid, (const float*)x, (const float*)w_gate_up,
                                sel, sel_w, top, n_real, ff, width, activation, act_param), "moe_gate_up");
    return 0;
}

extern "C" int rdl_moe_down_combine(void* out, int dtype, const void* mid, const void* x, const void* w_down, const int* sel,
                                    const float* sel_w, int n_rows, int top, int n_real, int ff, int width, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "moe_down_combine: bad dtype %d", dtype);
    RDL_REQUIRE(out && x && sel && ((mid && w_down) || n_real == 0) && top > 0 && width > 0, "moe_down_combine: bad arguments");
    if (n_rows == 0) return 0;
    RDL_REQUIRE(n_rows <= 65535, "moe_down_combine: %d rows exceed the grid limit", n_rows);
    const dim3 grid((width + PAIR_WARPS - 1) / PAIR_WARPS, n_rows);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == RDL_BF16)
        RDL_CHECK_EX(rdl_launch(moe_down_combine_kernel<__nv_bfloat16>, grid, dim3(PAIR_WARPS * 32), 0, st, (__nv_bfloat16*)out,
                                (const __nv_bfloat16*)mid, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_down, sel, sel_w, top, n_real, ff, width),
                     "moe_down_combine");
    else
        RDL_CHECK_EX(rdl_launch(moe_down_combine_kernel<float>, grid, dim3(PAIR_WARPS * 32), 0, st, (float*)out, (const float*)mid, (const float*)x,
                                (const float*)w_down, sel, sel_w, top, n_real, ff, width), "moe_down_combine");
    return 0;
}

extern "C" int rdl_moe_align(const int* sel, int n_pairs, int n_real, int max_tiles, int* pair_slot, int* slot_pair, int* tile_group,
                             void* stream) {
    RDL_REQUIRE(sel && pair_slot && slot_pair && tile_group && n_pairs > 0 && n_real > 0 && max_tiles > 0, "moe_align: bad arguments");
    RDL_REQUIRE((long long)max_tiles * MOE_TILE >= (long long)n_pairs + (long long)n_real * (MOE_TILE - 1),
                "moe_align: %d tiles cannot hold %d pairs of %d experts", max_tiles, n_pairs, n_real);
    RDL_REQUIRE(n_real <= 4096, "moe_align: %d experts exceed the 4,096 the kernel holds", n_real);
    const size_t smem = (3 * (size_t)n_real + 1) * sizeof(int);
    RDL_CHECK_EX(rdl_launch(moe_align_kernel, dim3(1), dim3(ALIGN_THREADS), smem, (cudaStream_t)stream, sel, n_pairs, n_real, max_tiles, pair_slot,
                            slot_pair, tile_group), "moe_align");
    return 0;
}

extern "C" int rdl_moe_gather(void* xs, const void* x, const int* slot_pair, const int* tile_group, const float* sel_w, int max_tiles,
                              int top, int width, void* stream) {
    RDL_REQUIRE(xs && x && slot_pair && tile_group && max_tiles > 0 && top > 0 && width > 0 && width % 8 == 0,
                "moe_gather: bad arguments (bfloat16 rows of a multiple of 8 values)");
    RDL_REQUIRE((uintptr_t)xs % 16 == 0 && (uintptr_t)x % 16 == 0, "moe_gather: rows must start on 16-byte boundaries");
    RDL_CHECK_EX(rdl_launch(moe_gather_kernel, dim3(max_tiles * MOE_TILE), dim3(128), 0, (cudaStream_t)stream, (uint4*)xs, (const uint4*)x, slot_pair,
                            tile_group, sel_w, top, width / 8), "moe_gather");
    return 0;
}

extern "C" int rdl_moe_combine(void* out, const void* y, const void* x, const int* pair_slot, const float* sel_w, int n_rows, int top,
                               int width, void* stream) {
    RDL_REQUIRE(out && y && x && pair_slot && n_rows > 0 && top > 0 && width > 0 && width % 8 == 0,
                "moe_combine: bad arguments (bfloat16 rows of a multiple of 8 values)");
    RDL_REQUIRE((uintptr_t)out % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)x % 16 == 0, "moe_combine: rows must start on 16-byte boundaries");
    RDL_CHECK_EX(rdl_launch(moe_combine_kernel, dim3(n_rows), dim3(128), 0, (cudaStream_t)stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)y,
                            (const __nv_bfloat16*)x, pair_slot, sel_w, top, width), "moe_combine");
    return 0;
}
