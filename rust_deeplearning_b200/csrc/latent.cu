// Kernels of the latent-attention mixer (keys and values compressed into one latent row per token).
//
// Per token the input projection leaves a packed row
//   [ q: heads x (dim unrotated | rot_dim rotated) | latent (kv_rank) | shared rotated key part (rot_dim) | ... ].
// What attention needs of it:
//   c   = latent / sqrt(mean(latent^2) + eps) * w           the latent, normed in float
//   kr  = R_p(shared key part),  q_rot <- R_p(q_rot)         R_p: rotation by the position's angles
// and the cache keeps ONE row [c | kr] per token, shared by all heads.  The score of head h is
//   (q_un[h] . W_uk[h] c  +  q_rot[h] . kr) * scale
// and its value row is W_uv[h] c.  Two ways of computing that are served here:
//   * expanded (whole prompts): k_un and v of every head come out of one product c [W_uk; W_uv]^T; rows
//     [Q | K | V] with heads padded to a common size are packed for the ordinary attention kernels
//     (rdl_latent_assemble);
//   * absorbed (single tokens, the 32-bit path): q'[h] = [W_uk[h]^T q_un[h] | q_rot[h]] attends over the cached rows
//     [c | kr] as keys and as values (one key/value head for all query heads), and head h's output is
//     W_uv[h] applied to the first kv_rank values of what comes out (rdl_heads_linear does both per-head
//     products; its epilogue can multiply by the output gate sigmoid(g[h])).
// Rotation pairs: interleaved (2i, 2i+1) or half-split (i, i + n/2), over the first `rot_n` dimensions of
// the rotated part; cos/sin come from float tables [position][rot_n / 2] (any scaling of frequencies or of
// the magnitude is in the tables).
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

template <typename T>
__device__ __forceinline__ void rotate_into(const T* src, T* dst, int n_rot, int total, int interleaved,
                                            const float* c, const float* s, int tid, int nthreads) {
    const int half = n_rot >> 1;
    for (int i = tid; i < half; i += nthreads) {
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        const float u = to_float(src[a]), v = to_float(src[b]);
        const float cs = c[i], sn = s[i];
        const float ru = u * cs - v * sn, rv = v * cs + u * sn;
        dst[a] = from_float<T>(ru);
        dst[b] = from_float<T>(rv);
    }
    if (dst != src)
        for (int i = n_rot + tid; i < total; i += nthreads) dst[i] = src[i];
}

// One block of LP_THREADS per token, whatever the step's row count: the order of the sum of squares depends on
// kv_rank alone.
constexpr int LP_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(LP_THREADS) latent_prepare_kernel(LatentPrepareArgs a) {
    __shared__ float red[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x;
    const int pos = a.tok_pos[t];
    if (pos < 0) return;                       // a padding row of a fixed-size batch
    T* row = (T*)a.rows + (long long)t * a.row_stride;
    const int half = a.rot_n >> 1;
    const float* cs = a.cos_t + (long long)pos * half;
    const float* sn = a.sin_t + (long long)pos * half;
    const int hq = a.dim + a.rot_dim;
    // queries: the rotated part of each head, in place or into the rows of the absorbed form; a work item is one
    // rotated pair, or one value of the part's unrotated tail that is only copied
    {
        const int tail = a.q_rot_out ? a.rot_dim - a.rot_n : 0, per_head = half + tail;
        for (int idx = threadIdx.x; idx < a.n_heads * per_head; idx += LP_THREADS) {
            const int h = idx / per_head, i = idx - h * per_head;
            const T* src = row + a.q_col + (long long)h * hq + a.dim;
            T* dst = a.q_rot_out ? (T*)a.q_rot_out + (long long)t * a.q_rot_stride + (long long)h * a.q_rot_head : (T*)src;
            if (i < half) {
                const int pa = a.interleaved ? 2 * i : i, pb = a.interleaved ? 2 * i + 1 : i + half;
                const float u = to_float(src[pa]), v = to_float(src[pb]);
                dst[pa] = from_float<T>(u * cs[i] - v * sn[i]);
                dst[pb] = from_float<T>(v * cs[i] + u * sn[i]);
            } else {
                dst[a.rot_n + i - half] = src[a.rot_n + i - half];
            }
        }
    }
    if (a.latent_col < 0) return;              // a layer that reads another layer's latent rows
    // the latent: root mean square in float, a fixed order of additions
    const T* lat = row + a.latent_col;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.kv_rank; i += LP_THREADS) {
        const float v = to_float(lat[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)a.kv_rank + a.eps);
    T* out = (T*)a.latent_out + (long long)t * (a.kv_rank + a.rot_dim);
    for (int i = threadIdx.x; i < a.kv_rank; i += LP_THREADS)
        out[i] = from_float<T>(to_float(lat[i]) * inv * rdl_load(a.norm_w, i, a.norm_w_dtype));
    rotate_into<T>(lat + a.kv_rank, out + a.kv_rank, a.rot_n, a.rot_dim, a.interleaved, cs, sn, threadIdx.x, LP_THREADS);
    if (!a.do_write) return;
    const int seq = a.tok_seq[t];
    // In a ring a later token of this step may land on the same row: only the last writer writes.
    if ((long long)pos + (long long)a.ring_pages * a.page_size < (long long)a.seq_end[seq]) return;
    __syncthreads();                           // the row [c | kr] is complete
    const int width = a.kv_rank + a.rot_dim;
    T* dst = (T*)a.cache + rdl_cache_offset(a.tables + (long long)seq * a.table_width, pos, a.page_size, a.ring_pages, 1, 0, width);
    const int r = pos % a.page_size;           // chunks of a cache row are stored swizzled by its place in the page
    for (int i = threadIdx.x; i < width; i += LP_THREADS) dst[rdl_cache_col<T>(r, i, width)] = out[i];
}

// The same work in bfloat16 with 16-byte accesses, where every size and offset is a whole number of 8-value chunks: with
// interleaved pairs a chunk of the rotated parts holds four whole pairs; with half-split pairs (rot_n a multiple of 16)
// chunk c of the first half turns together with chunk c + rot_n / 16 of the second.  A chunk of the latent goes to the
// rows and to its (swizzled) place in the cache as soon as it is normed.  The sum of squares is formed chunk by chunk, then by the block's
// fixed tree: its order depends on kv_rank alone.
__device__ __forceinline__ uint4 rotate_chunk(const uint4 raw, const float* __restrict__ cs, const float* __restrict__ sn) {
    const float4 c4 = *reinterpret_cast<const float4*>(cs), s4 = *reinterpret_cast<const float4*>(sn);
    const float c[4] = {c4.x, c4.y, c4.z, c4.w}, s[4] = {s4.x, s4.y, s4.z, s4.w};
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint4 out;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h[i]);
        o[i] = __floats2bfloat162_rn(v.x * c[i] - v.y * s[i], v.y * c[i] + v.x * s[i]);
    }
    return out;
}

// half-split pairs: value i of chunk `lo` turns with value i of chunk `hi` by the eight angles at cs, sn
__device__ __forceinline__ void rotate_half_chunks(uint4& lo, uint4& hi, const float* __restrict__ cs, const float* __restrict__ sn) {
    const float4 c0 = *reinterpret_cast<const float4*>(cs), c1 = *reinterpret_cast<const float4*>(cs + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sn), s1 = *reinterpret_cast<const float4*>(sn + 4);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w}, s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    __nv_bfloat162* u = reinterpret_cast<__nv_bfloat162*>(&lo);
    __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(u[i]), y = __bfloat1622float2(v[i]);
        u[i] = __floats2bfloat162_rn(x.x * c[2 * i] - y.x * s[2 * i], x.y * c[2 * i + 1] - y.y * s[2 * i + 1]);
        v[i] = __floats2bfloat162_rn(y.x * c[2 * i] + x.x * s[2 * i], y.y * c[2 * i + 1] + x.y * s[2 * i + 1]);
    }
}

__global__ void __launch_bounds__(LP_THREADS) latent_prepare_vec_kernel(LatentPrepareArgs a) {
    __shared__ float red[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x;
    const int pos = a.tok_pos[t];
    if (pos < 0) return;                       // a padding row of a fixed-size batch
    typedef __nv_bfloat16 T;
    T* row = (T*)a.rows + (long long)t * a.row_stride;
    const int half = a.rot_n >> 1;
    const float* cs = a.cos_t + (long long)pos * half;
    const float* sn = a.sin_t + (long long)pos * half;
    const int hq = a.dim + a.rot_dim, rc = a.rot_dim >> 3, rot_chunks = a.rot_n >> 3;
    const int hcn = a.interleaved ? 0 : rot_chunks >> 1;      // half-split pairs: chunk c turns with chunk c + hcn
    // queries: chunk c of head h's rotated part (half-split pairs: a work item holds both chunks of a pair)
    const int q_items = rc - hcn;
    for (int idx = threadIdx.x; idx < a.n_heads * q_items; idx += LP_THREADS) {
        const int h = idx / q_items, j = idx - h * q_items;
        const int c = j < hcn ? j : j + hcn;
        T* src = row + a.q_col + (long long)h * hq + a.dim + c * 8;
        T* dst = a.q_rot_out ? (T*)a.q_rot_out + (long long)t * a.q_rot_stride + (long long)h * a.q_rot_head + c * 8 : src;
        uint4 v = *reinterpret_cast<const uint4*>(src);
        if (j < hcn) {
            uint4 w = *reinterpret_cast<const uint4*>(src + hcn * 8);
            rotate_half_chunks(v, w, cs + c * 8, sn + c * 8);
            *reinterpret_cast<uint4*>(dst + hcn * 8) = w;
        } else if (a.interleaved && c < rot_chunks) {
            v = rotate_chunk(v, cs + c * 4, sn + c * 4);
        } else if (dst == src) {
            continue;
        }
        *reinterpret_cast<uint4*>(dst) = v;
    }
    if (a.latent_col < 0) return;              // a layer that reads another layer's latent rows
    const T* lat = row + a.latent_col;
    const int lc = a.kv_rank >> 3, width = a.kv_rank + a.rot_dim, chunks = width >> 3;
    float ss = 0.f;
    for (int c = threadIdx.x; c < lc; c += LP_THREADS) {
        const uint4 raw = *reinterpret_cast<const uint4*>(lat + c * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __bfloat1622float2(h[i]);
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
        }
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)a.kv_rank + a.eps);
    T* out = (T*)a.latent_out + (long long)t * width;
    // where the row goes in the cache (in a ring a later token of this step may land on the same row: only the last writes)
    T* cache_row = nullptr;
    int r = 0;
    if (a.do_write) {
        const int seq = a.tok_seq[t];
        if ((long long)pos + (long long)a.ring_pages * a.page_size >= (long long)a.seq_end[seq]) {
            cache_row = (T*)a.cache + rdl_cache_offset(a.tables + (long long)seq * a.table_width, pos, a.page_size, a.ring_pages, 1, 0, width);
            r = pos % a.page_size;
        }
    }
    for (int c = threadIdx.x; c < chunks; c += LP_THREADS) {
        uint4 v = *reinterpret_cast<const uint4*>(lat + c * 8);
        if (c < lc) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
            uint4 res;
            __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 x = __bfloat1622float2(h[i]);
                o[i] = __floats2bfloat162_rn(x.x * inv * rdl_load(a.norm_w, c * 8 + 2 * i, a.norm_w_dtype),
                                             x.y * inv * rdl_load(a.norm_w, c * 8 + 2 * i + 1, a.norm_w_dtype));
            }
            v = res;
        } else if (a.interleaved && c - lc < rot_chunks) {
            v = rotate_chunk(v, cs + (c - lc) * 4, sn + (c - lc) * 4);
        } else if (c - lc < hcn) {             // half-split pairs: this chunk and its partner, both stored here
            uint4 w = *reinterpret_cast<const uint4*>(lat + (c + hcn) * 8);
            rotate_half_chunks(v, w, cs + (c - lc) * 8, sn + (c - lc) * 8);
            *reinterpret_cast<uint4*>(out + (c + hcn) * 8) = w;
            if (cache_row) *reinterpret_cast<uint4*>(cache_row + rdl_swizzled_chunk(r, c + hcn, chunks) * 8) = w;
        } else if (c - lc < 2 * hcn) {
            continue;                          // stored by its partner's thread
        }
        *reinterpret_cast<uint4*>(out + c * 8) = v;
        if (cache_row) *reinterpret_cast<uint4*>(cache_row + rdl_swizzled_chunk(r, c, chunks) * 8) = v;
    }
}

// A step's latent rows [c | kr] into the cache, as a kernel of its own (a ring group's write that had to wait
// for the readers of the rows it overwrites).
template <typename T>
__global__ void latent_write_kernel(LatentPrepareArgs a) {
    const int t = blockIdx.x;
    const int pos = a.tok_pos[t];
    if (pos < 0) return;
    const int seq = a.tok_seq[t];
    if ((long long)pos + (long long)a.ring_pages * a.page_size < (long long)a.seq_end[seq]) return;
    const int width = a.kv_rank + a.rot_dim;
    const T* src = (const T*)a.latent_out + (long long)t * width;
    T* dst = (T*)a.cache + rdl_cache_offset(a.tables + (long long)seq * a.table_width, pos, a.page_size, a.ring_pages, 1, 0, width);
    const int r = pos % a.page_size;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[rdl_cache_col<T>(r, i, width)] = src[i];
}

// Packed rows [Q | K | V] for the ordinary attention kernels, heads padded with zeros to `pad` values:
//   Q[h] = [q_un[h] | q_rot[h] (rotated)], K[h] = [k_un[h] | kr], V[h] = v[h]
// q from the projection's rows, k_un and v from the product c [W_uk; W_uv]^T ([tokens, H dim + H vdim]),
// kr from the latent rows [c | kr].
template <typename T>
__global__ void latent_assemble_kernel(T* __restrict__ out, const T* __restrict__ rows, long long row_stride, int q_col,
                                       const T* __restrict__ kv, const T* __restrict__ latent, int n_heads, int dim, int rot_dim,
                                       int vdim, int kv_rank, int pad) {
    const int t = blockIdx.x;
    const int hq = dim + rot_dim;
    const long long width = 3LL * n_heads * pad;
    T* o = out + (long long)t * width;
    const T* q = rows + (long long)t * row_stride + q_col;
    const T* kvr = kv + (long long)t * n_heads * (dim + vdim);
    const T* kr = latent + (long long)t * (kv_rank + rot_dim) + kv_rank;
    const int per = n_heads * pad;
    for (int i = threadIdx.x; i < 3 * per; i += blockDim.x) {
        const int part = i / per, j = i - part * per, h = j / pad, e = j - h * pad;
        T v = from_float<T>(0.f);
        if (part == 0) {
            if (e < hq) v = q[(long long)h * hq + e];
        } else if (part == 1) {
            if (e < dim) v = kvr[(long long)h * dim + e];
            else if (e < hq) v = kr[e - dim];
        } else {
            if (e < vdim) v = kvr[(long long)n_heads * dim + (long long)h * vdim + e];
        }
        o[i] = v;
    }
}

// The same in 16-byte pieces of PIECE values, where every size is a whole number of pieces and every row starts on a
// 16-byte boundary: a grid-stride loop over the pieces of all tokens.
template <typename T>
__global__ void latent_assemble_vec_kernel(uint4* __restrict__ out, const T* __restrict__ rows, long long row_stride, int q_col,
                                           const T* __restrict__ kv, const T* __restrict__ latent, int n_tokens, int n_heads, int dim,
                                           int rot_dim, int vdim, int kv_rank, int pad) {
    constexpr int PIECE = 16 / (int)sizeof(T);
    const int hq = dim + rot_dim, pp = pad / PIECE, per = n_heads * pp;
    const long long total = 3LL * per * n_tokens;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(idx / (3 * per)), i = (int)(idx - (long long)t * 3 * per);
        const int part = i / per, j = i - part * per, h = j / pp, e = (j - h * pp) * PIECE;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (part == 0) {
            if (e < hq) v = *reinterpret_cast<const uint4*>(rows + (long long)t * row_stride + q_col + (long long)h * hq + e);
        } else if (part == 1) {
            if (e < dim) v = *reinterpret_cast<const uint4*>(kv + (long long)t * n_heads * (dim + vdim) + (long long)h * dim + e);
            else if (e < hq) v = *reinterpret_cast<const uint4*>(latent + (long long)t * (kv_rank + rot_dim) + kv_rank + e - dim);
        } else {
            if (e < vdim) v = *reinterpret_cast<const uint4*>(kv + (long long)t * n_heads * (dim + vdim) + (long long)n_heads * dim + (long long)h * vdim + e);
        }
        out[idx] = v;
    }
}

// out[t, h, :vdim] = in[t, h, :vdim] * sigmoid(g[t, h]) in 16-byte pieces of bfloat16 (g_elem: a gate per value,
// g[t, h * vdim + i], read in 16-byte pieces too when g_vec)
__global__ void gate_heads_vec_kernel(uint4* __restrict__ out, const __nv_bfloat16* __restrict__ in, long long in_stride, int in_head,
                                      const __nv_bfloat16* __restrict__ g, long long g_stride, int n_tokens, int n_heads, int vdim,
                                      int g_elem, int g_vec) {
    const int vp = vdim / 8;
    const long long total = (long long)n_tokens * n_heads * vp;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(idx / (n_heads * vp)), j = (int)(idx - (long long)t * n_heads * vp), h = j / vp, e = (j - h * vp) * 8;
        float gate[8];
        if (g_elem) {
            const __nv_bfloat16* gp = g + (long long)t * g_stride + (long long)h * vdim + e;
            if (g_vec) {
                const uint4 graw = *reinterpret_cast<const uint4*>(gp);
                const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&graw);
#pragma unroll
                for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(gh[i]); gate[2 * i] = v.x; gate[2 * i + 1] = v.y; }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) gate[i] = __bfloat162float(gp[i]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) gate[i] = 1.0f / (1.0f + expf(-gate[i]));
        } else {
            const float one = 1.0f / (1.0f + expf(-__bfloat162float(g[(long long)t * g_stride + h])));
#pragma unroll
            for (int i = 0; i < 8; ++i) gate[i] = one;
        }
        const uint4 raw = *reinterpret_cast<const uint4*>(in + (long long)t * in_stride + (long long)h * in_head + e);
        const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&raw);
        uint4 res;
        __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __bfloat1622float2(hp[i]);
            rp[i] = __floats2bfloat162_rn(v.x * gate[2 * i], v.y * gate[2 * i + 1]);
        }
        out[idx] = res;
    }
}

// out[t, h, i] = in[t, h, i] * sigmoid(g[t, h]) for i < vdim: the output gate on the heads of an attention result
// (g_elem: a gate per value, g[t, h * vdim + i]).
template <typename T>
__global__ void gate_heads_kernel(T* __restrict__ out, const T* __restrict__ in, long long in_stride, int in_head,
                                  const T* __restrict__ g, long long g_stride, int n_heads, int vdim, int g_elem) {
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < n_heads * vdim; i += blockDim.x) {
        const int h = i / vdim, e = i - h * vdim;
        const float gate = 1.0f / (1.0f + expf(-to_float(g[(long long)t * g_stride + (g_elem ? i : h)])));
        out[(long long)t * n_heads * vdim + i] = from_float<T>(to_float(in[(long long)t * in_stride + (long long)h * in_head + e]) * gate);
    }
}

// out[t, h, j] = sum_k w[h, j, k] x[t, h, k]  (times sigmoid(g[t, h]), or of g[t, h * n_out + j] with gate_elem, if g is given): a product per head.
// One warp per (token, head, 32 consecutive j)?  No: a warp per (token tile, head, j) would re-read x; here a warp
// takes one (head, j) for HL_ROWS tokens, lanes split k, so a weight row is read once for those tokens.  The sum
// over k runs lane by lane in a fixed order and ends in a shuffle tree: it depends on k alone.
constexpr int HL_ROWS = 8, HL_WARPS = 8;

__device__ __forceinline__ void load_piece(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(h[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
}
__device__ __forceinline__ void load_piece(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}

template <typename T>
__global__ void __launch_bounds__(HL_WARPS * 32) heads_linear_kernel(HeadsLinearArgs a) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, t0 = blockIdx.z * HL_ROWS;
    const int j = blockIdx.x * HL_WARPS + warp;
    if (j >= a.n_out) return;
    const T* w = (const T*)a.w + ((long long)h * a.n_out + j) * a.k;
    float acc[HL_ROWS];
#pragma unroll
    for (int r = 0; r < HL_ROWS; ++r) acc[r] = 0.f;
    const int rows = min(HL_ROWS, a.n_tokens - t0);
    const T* xb = (const T*)a.x + (long long)t0 * a.x_stride + (long long)h * a.x_head;
    constexpr int N = 16 / (int)sizeof(T);       // values of a 16-byte piece
    // 16-byte pieces where every row of w and x starts on such a boundary; which form runs depends on sizes and addresses, not on the row count
    if (a.k % N == 0 && (((uintptr_t)a.w | (uintptr_t)a.x) & 15) == 0 && a.x_stride % N == 0 && a.x_head % N == 0) {
        for (int k = lane * N; k < a.k; k += 32 * N) {
            float wv[N];
            load_piece(w + k, wv);
#pragma unroll
            for (int r = 0; r < HL_ROWS; ++r) {
                if (r < rows) {
                    float xv[N];
                    load_piece(xb + (long long)r * a.x_stride + k, xv);
#pragma unroll
                    for (int j2 = 0; j2 < N; ++j2) acc[r] = fmaf(wv[j2], xv[j2], acc[r]);
                }
            }
        }
    } else {
        for (int k = lane; k < a.k; k += 32) {
            const float wv = to_float(w[k]);
#pragma unroll
            for (int r = 0; r < HL_ROWS; ++r)
                if (r < rows) acc[r] = fmaf(wv, to_float(xb[(long long)r * a.x_stride + k]), acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < HL_ROWS; ++r) {
        if (r >= rows) break;
        float v = warp_sum(acc[r]);
        if (lane == 0) {
            if (a.gate) v *= 1.0f / (1.0f + expf(-to_float(((const T*)a.gate)[(long long)(t0 + r) * a.gate_stride + (a.gate_elem ? h * a.n_out + j : h)])));
            ((T*)a.out)[(long long)(t0 + r) * a.out_stride + (long long)h * a.out_head + j] = from_float<T>(v);
        }
    }
}

}  // namespace

extern "C" int rdl_latent_prepare(const LatentPrepareArgs* a, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(a->dtype), "latent_prepare: bad dtype %d", a->dtype);
    RDL_REQUIRE(a->n_tokens >= 0 && a->n_heads > 0 && a->dim >= 0 && a->rot_dim > 0 && a->kv_rank > 0, "latent_prepare: bad sizes");
    RDL_REQUIRE(a->rot_n >= 0 && a->rot_n % 2 == 0 && a->rot_n <= a->rot_dim, "latent_prepare: %d rotated dimensions do not fit a part of %d", a->rot_n, a->rot_dim);
    RDL_REQUIRE(a->rows && a->tok_pos && (a->rot_n == 0 || (a->cos_t && a->sin_t)), "latent_prepare: missing rows, positions or tables");
    RDL_REQUIRE(a->latent_col < 0 || (a->latent_out && a->norm_w), "latent_prepare: missing latent output or norm weight");
    RDL_REQUIRE(!a->do_write || (a->latent_col >= 0 && a->cache && a->tables && a->tok_seq && a->seq_end && a->page_size > 0 && a->ring_pages > 0 &&
                                 a->ring_pages <= a->table_width), "latent_prepare: cache write without storage or with bad paging");
    if (a->n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const bool chunked = a->dtype == RDL_BF16 && a->rot_n % (a->interleaved ? 8 : 16) == 0 && a->dim % 8 == 0 && a->rot_dim % 8 == 0 && a->kv_rank % 8 == 0 &&
                         a->q_col % 8 == 0 && a->row_stride % 8 == 0 && ((uintptr_t)a->rows & 15) == 0 && (a->latent_col < 0 || a->latent_col % 8 == 0) &&
                         (!a->q_rot_out || (((uintptr_t)a->q_rot_out & 15) == 0 && a->q_rot_stride % 8 == 0 && a->q_rot_head % 8 == 0)) &&
                         (a->latent_col < 0 || ((uintptr_t)a->latent_out & 15) == 0) && (!a->do_write || ((uintptr_t)a->cache & 15) == 0) &&
                         (a->rot_n == 0 || (((uintptr_t)a->cos_t | (uintptr_t)a->sin_t) & 15) == 0);
    if (chunked)
        RDL_CHECK_EX(rdl_launch(latent_prepare_vec_kernel, dim3(a->n_tokens), dim3(LP_THREADS), 0, st, *a), "latent_prepare");
    else if (a->dtype == RDL_BF16)
        RDL_CHECK_EX(rdl_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(a->n_tokens), dim3(LP_THREADS), 0, st, *a), "latent_prepare");
    else
        RDL_CHECK_EX(rdl_launch(latent_prepare_kernel<float>, dim3(a->n_tokens), dim3(LP_THREADS), 0, st, *a), "latent_prepare");
    return 0;
}

extern "C" int rdl_latent_write(const LatentPrepareArgs* a, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(a->dtype), "latent_write: bad dtype %d", a->dtype);
    RDL_REQUIRE(a->latent_out && a->cache && a->tables && a->tok_seq && a->tok_pos && a->seq_end && a->page_size > 0 && a->ring_pages > 0 &&
                a->ring_pages <= a->table_width, "latent_write: missing rows, storage or paging");
    if (a->n_tokens == 0) return 0;
    if (a->dtype == RDL_BF16)
        latent_write_kernel<__nv_bfloat16><<<a->n_tokens, 128, 0, (cudaStream_t)stream>>>(*a);
    else
        latent_write_kernel<float><<<a->n_tokens, 128, 0, (cudaStream_t)stream>>>(*a);
    RDL_CHECK_LAUNCH("latent_write");
    return 0;
}

extern "C" int rdl_latent_assemble(void* out, int dtype, const void* rows, long long row_stride, int q_col, const void* kv,
                                   const void* latent, int n_tokens, int n_heads, int dim, int rot_dim, int vdim, int kv_rank,
                                   int pad, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "latent_assemble: bad dtype %d", dtype);
    RDL_REQUIRE(out && rows && kv && latent && n_heads > 0 && pad >= dim + rot_dim && pad >= vdim, "latent_assemble: bad arguments");
    if (n_tokens == 0) return 0;
    const int piece = dtype == RDL_BF16 ? 8 : 4;
    if (dim % piece == 0 && rot_dim % piece == 0 && vdim % piece == 0 && pad % piece == 0 && kv_rank % piece == 0 && row_stride % piece == 0 &&
        q_col % piece == 0 && (((uintptr_t)out | (uintptr_t)rows | (uintptr_t)kv | (uintptr_t)latent) & 15) == 0) {
        const long long total = 3LL * n_heads * (pad / piece) * n_tokens;
        const long long want = (total + 255) / 256;
        const unsigned blocks = (unsigned)(want > (long long)rdl_sm_count() * 16 ? (long long)rdl_sm_count() * 16 : want);
        if (dtype == RDL_BF16)
            latent_assemble_vec_kernel<__nv_bfloat16><<<blocks, 256, 0, (cudaStream_t)stream>>>(
                (uint4*)out, (const __nv_bfloat16*)rows, row_stride, q_col, (const __nv_bfloat16*)kv, (const __nv_bfloat16*)latent, n_tokens,
                n_heads, dim, rot_dim, vdim, kv_rank, pad);
        else
            latent_assemble_vec_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((uint4*)out, (const float*)rows, row_stride, q_col,
                                                                                         (const float*)kv, (const float*)latent, n_tokens,
                                                                                         n_heads, dim, rot_dim, vdim, kv_rank, pad);
        RDL_CHECK_LAUNCH("latent_assemble");
        return 0;
    }
    if (dtype == RDL_BF16)
        latent_assemble_kernel<__nv_bfloat16><<<n_tokens, 256, 0, (cudaStream_t)stream>>>(
            (__nv_bfloat16*)out, (const __nv_bfloat16*)rows, row_stride, q_col, (const __nv_bfloat16*)kv, (const __nv_bfloat16*)latent,
            n_heads, dim, rot_dim, vdim, kv_rank, pad);
    else
        latent_assemble_kernel<float><<<n_tokens, 256, 0, (cudaStream_t)stream>>>((float*)out, (const float*)rows, row_stride, q_col,
                                                                                   (const float*)kv, (const float*)latent, n_heads, dim,
                                                                                   rot_dim, vdim, kv_rank, pad);
    RDL_CHECK_LAUNCH("latent_assemble");
    return 0;
}

extern "C" int rdl_gate_heads(void* out, int dtype, const void* in, long long in_stride, int in_head, const void* g, long long g_stride,
                              int n_tokens, int n_heads, int vdim, int g_elem, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "gate_heads: bad dtype %d", dtype);
    RDL_REQUIRE(out && in && g && n_heads > 0 && vdim > 0 && in_head >= vdim, "gate_heads: bad arguments");
    if (n_tokens == 0) return 0;
    if (dtype == RDL_BF16 && vdim % 8 == 0 && in_head % 8 == 0 && in_stride % 8 == 0 && (((uintptr_t)out | (uintptr_t)in) & 15) == 0) {
        const long long want = ((long long)n_tokens * n_heads * (vdim / 8) + 255) / 256;
        const unsigned blocks = (unsigned)(want > (long long)rdl_sm_count() * 16 ? (long long)rdl_sm_count() * 16 : want);
        gate_heads_vec_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((uint4*)out, (const __nv_bfloat16*)in, in_stride, in_head,
                                                                         (const __nv_bfloat16*)g, g_stride, n_tokens, n_heads, vdim, g_elem,
                                                                         (int)(g_elem && g_stride % 8 == 0 && ((uintptr_t)g & 15) == 0));
        RDL_CHECK_LAUNCH("gate_heads");
        return 0;
    }
    if (dtype == RDL_BF16)
        gate_heads_kernel<__nv_bfloat16><<<n_tokens, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)in, in_stride, in_head,
                                                                                      (const __nv_bfloat16*)g, g_stride, n_heads, vdim, g_elem);
    else
        gate_heads_kernel<float><<<n_tokens, 256, 0, (cudaStream_t)stream>>>((float*)out, (const float*)in, in_stride, in_head, (const float*)g,
                                                                              g_stride, n_heads, vdim, g_elem);
    RDL_CHECK_LAUNCH("gate_heads");
    return 0;
}

extern "C" int rdl_heads_linear(const HeadsLinearArgs* a, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(a->dtype), "heads_linear: bad dtype %d", a->dtype);
    RDL_REQUIRE(a->out && a->x && a->w && a->n_heads > 0 && a->n_out > 0 && a->k > 0 && a->n_tokens >= 0, "heads_linear: bad arguments");
    RDL_REQUIRE(a->n_heads <= 65535, "heads_linear: %d heads exceed the grid limit", a->n_heads);
    if (a->n_tokens == 0) return 0;
    const dim3 grid((a->n_out + HL_WARPS - 1) / HL_WARPS, a->n_heads, (a->n_tokens + HL_ROWS - 1) / HL_ROWS);
    RDL_REQUIRE(grid.z <= 65535, "heads_linear: %d rows exceed the grid limit", a->n_tokens);
    cudaStream_t st = (cudaStream_t)stream;
    if (a->dtype == RDL_BF16)
        RDL_CHECK_EX(rdl_launch(heads_linear_kernel<__nv_bfloat16>, grid, dim3(HL_WARPS * 32), 0, st, *a), "heads_linear");
    else
        RDL_CHECK_EX(rdl_launch(heads_linear_kernel<float>, grid, dim3(HL_WARPS * 32), 0, st, *a), "heads_linear");
    return 0;
}
