// Rotary position encoding of the query and key heads of a packed [tokens, heads, head_dim]
// buffer, in place, and the write of the new key and value rows into a paged cache.
//
// Rotation (reference: rustml/nn/main/src/core/rope.rs:188-191, half-split pairing):
//   out[i]        = x[i] * cos - x[i + r/2] * sin
//   out[i + r/2]  = x[i] * sin + x[i + r/2] * cos      for i < r/2, r = rotary_dim
// with cos/sin read from float tables [position][r/2]; the product is formed in float.
// The cache write corresponds to rustml/nn/main/src/core/kv_cache.rs:97-109, with pages and a
// length per sequence instead of one shared length.
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, int n_heads, int n_kv_heads, int head_dim, int rotary_dim,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                  int do_rope, int do_write, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  const int* __restrict__ tables, int table_width, int page_size, int ring_pages,
                                  const int* __restrict__ seq_end) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x;
    const int head = blockIdx.y;
    const int total_heads = n_heads + 2 * n_kv_heads;
    T* row = qkv + ((long long)t * total_heads + head) * head_dim;
    const int pos = tok_pos[t];
    if (pos < 0) return;  // a padding row of a fixed-size batch
    const bool is_v = head >= n_heads + n_kv_heads;

    if (do_rope && !is_v) {
        const int half = rotary_dim >> 1;
        const float* c = cos_t + (long long)pos * half;
        const float* s = sin_t + (long long)pos * half;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float x1 = to_float(row[i]), x2 = to_float(row[i + half]);
            const float cs = c[i], sn = s[i];
            row[i] = from_float<T>(x1 * cs - x2 * sn);
            row[i + half] = from_float<T>(x1 * sn + x2 * cs);
        }
    }
    if (!do_write || head < n_heads) return;
    const int seq = tok_seq[t];
    // In a ring a later token of this step may land on the same row: only the last writer writes.
    const long long ring_rows = (long long)ring_pages * page_size;
    if ((long long)pos + ring_rows < (long long)seq_end[seq]) return;
    __syncthreads();  // the rotated key of this block is complete
    const int kv_head = is_v ? head - n_heads - n_kv_heads : head - n_heads;
    T* dst = (is_v ? v_cache : k_cache) +
             rdl_cache_offset(tables + (long long)seq * table_width, pos, page_size, ring_pages, n_kv_heads, kv_head, head_dim);
    const int r = pos % page_size;   // chunks of a cache row are stored swizzled by its place in the page
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) dst[rdl_cache_col<T>(r, i, head_dim)] = row[i];
}

// The same work with 16-byte accesses: one block per token, a thread per 16-byte chunk (or pair of
// chunks that rotate together).  Used when head_dim and rotary_dim / 2 are whole numbers of chunks.
template <typename T> struct Chunk;
template <> struct Chunk<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(h[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
    }
    static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        return raw;
    }
};
template <> struct Chunk<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    static __device__ __forceinline__ uint4 pack(const float (&f)[4]) {
        uint4 raw;
        raw.x = __float_as_uint(f[0]); raw.y = __float_as_uint(f[1]); raw.z = __float_as_uint(f[2]); raw.w = __float_as_uint(f[3]);
        return raw;
    }
};

template <typename T>
__global__ void __launch_bounds__(256) rope_cache_vec_kernel(T* __restrict__ qkv, int n_heads, int n_kv_heads, int head_dim, int rotary_dim,
                                                             const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                             const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                                             int do_rope, int do_write, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                             const int* __restrict__ tables, int table_width, int page_size,
                                                             int ring_pages, const int* __restrict__ seq_end) {
    constexpr int N = Chunk<T>::N;
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    if (pos < 0) return;  // a padding row of a fixed-size batch
    const int total_heads = n_heads + 2 * n_kv_heads;
    const int chunks = head_dim / N;
    const int half = rotary_dim >> 1, half_chunks = do_rope ? half / N : 0;
    T* base = qkv + (long long)t * total_heads * head_dim;
    bool write = do_write && n_kv_heads > 0;
    int r = 0;
    long long page_base = 0;
    if (write) {
        const int seq = tok_seq[t];
        // In a ring a later token of this step may land on the same row: only the last writer writes.
        if ((long long)pos + (long long)ring_pages * page_size < (long long)seq_end[seq]) write = false;
        const int logical = pos / page_size;
        r = pos - logical * page_size;
        page_base = (long long)tables[(long long)seq * table_width + logical % ring_pages] * n_kv_heads;
    }
    // Work items, one 16-byte chunk of output pair or chunk each, so that no thread idles: first the rotated
    // pairs (chunk c with chunk c + half) of the query and key heads, then the chunks that are only copied
    // to the cache: the unrotated tail of the key heads and the value heads.
    const int n_pairs = (n_heads + n_kv_heads) * half_chunks;
    const int k_tail = chunks - 2 * half_chunks;                  // unrotated chunks of a key head
    const int n_copy = write ? n_kv_heads * (k_tail + chunks) : 0;
    for (int item = threadIdx.x; item < n_pairs + n_copy; item += blockDim.x) {
        int head, c;
        bool rotated = item < n_pairs;
        if (rotated) {
            head = item / half_chunks;
            c = item - head * half_chunks;
        } else {
            const int rest = item - n_pairs;
            if (rest < n_kv_heads * k_tail) {
                head = n_heads + rest / k_tail;
                c = 2 * half_chunks + rest % k_tail;
            } else {
                const int v = rest - n_kv_heads * k_tail;
                head = n_heads + n_kv_heads + v / chunks;
                c = v % chunks;
            }
        }
        const bool is_q = head < n_heads, is_v = head >= n_heads + n_kv_heads;
        T* row = base + (long long)head * head_dim;
        T* dst = nullptr;
        if (write && !is_q) {
            const int kv_head = is_v ? head - n_heads - n_kv_heads : head - n_heads;
            dst = (is_v ? v_cache : k_cache) + ((page_base + kv_head) * page_size + r) * head_dim;
        }
        float a[N];
        Chunk<T>::load(row + c * N, a);
        if (rotated) {
            float b[N], cs[N], sn[N];
            Chunk<T>::load(row + (c + half_chunks) * N, b);
            const float4* cp = reinterpret_cast<const float4*>(cos_t + (long long)pos * half + c * N);
            const float4* sp = reinterpret_cast<const float4*>(sin_t + (long long)pos * half + c * N);
#pragma unroll
            for (int i = 0; i < N / 4; ++i) {
                const float4 cv = __ldg(cp + i), sv = __ldg(sp + i);
                cs[4 * i] = cv.x; cs[4 * i + 1] = cv.y; cs[4 * i + 2] = cv.z; cs[4 * i + 3] = cv.w;
                sn[4 * i] = sv.x; sn[4 * i + 1] = sv.y; sn[4 * i + 2] = sv.z; sn[4 * i + 3] = sv.w;
            }
            float lo[N], hi[N];
#pragma unroll
            for (int i = 0; i < N; ++i) {
                lo[i] = a[i] * cs[i] - b[i] * sn[i];
                hi[i] = a[i] * sn[i] + b[i] * cs[i];
            }
            const uint4 plo = Chunk<T>::pack(lo), phi = Chunk<T>::pack(hi);
            *reinterpret_cast<uint4*>(row + c * N) = plo;
            *reinterpret_cast<uint4*>(row + (c + half_chunks) * N) = phi;
            if (dst) {
                *reinterpret_cast<uint4*>(dst + rdl_swizzled_chunk(r, c, chunks) * N) = plo;
                *reinterpret_cast<uint4*>(dst + rdl_swizzled_chunk(r, c + half_chunks, chunks) * N) = phi;
            }
        } else if (dst) {
            *reinterpret_cast<uint4*>(dst + rdl_swizzled_chunk(r, c, chunks) * N) = Chunk<T>::pack(a);
        }
    }
}

extern "C" int rdl_rope_cache(void* qkv, int dtype, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                              int rotary_dim, const float* cos_table, const float* sin_table,
                              const int* tok_seq, const int* tok_pos, int do_rope, int do_write,
                              void* k_cache, void* v_cache, const int* tables, int table_width, int page_size,
                              int ring_pages, const int* seq_end, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "rope_cache: bad dtype %d", dtype);
    RDL_REQUIRE(n_tokens >= 0 && n_heads >= 0 && n_kv_heads >= 0 && n_heads + n_kv_heads > 0 && head_dim > 0,
                "rope_cache: bad sizes tokens=%d heads=%d kv_heads=%d head_dim=%d", n_tokens, n_heads, n_kv_heads, head_dim);
    RDL_REQUIRE(!do_rope || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim && cos_table && sin_table),
                "rope_cache: rotary_dim %d must be even and at most head_dim %d", rotary_dim, head_dim);
    RDL_REQUIRE(!do_write || n_kv_heads == 0 ||
                    (k_cache && v_cache && tables && seq_end && tok_seq && page_size > 0 && ring_pages > 0 && ring_pages <= table_width),
                "rope_cache: cache write needs storage, page tables and lengths (page_size=%d ring_pages=%d table_width=%d)",
                page_size, ring_pages, table_width);
    const int total_heads = n_heads + 2 * n_kv_heads;
    RDL_REQUIRE(total_heads <= 65535, "rope_cache: %d heads exceed the grid limit", total_heads);
    if (n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    const int per_chunk = dtype == RDL_BF16 ? 8 : 4;
    const bool aligned = ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 &&
                         ((uintptr_t)cos_table & 15) == 0 && ((uintptr_t)sin_table & 15) == 0;
    if (aligned && head_dim % per_chunk == 0 && (!do_rope || (rotary_dim / 2) % per_chunk == 0)) {
        // two work items a thread where there are many (the kernel's comment says what an item is)
        const int chunks = head_dim / per_chunk, half_chunks = do_rope ? rotary_dim / 2 / per_chunk : 0;
        const int items = (n_heads + n_kv_heads) * half_chunks + n_kv_heads * (2 * chunks - 2 * half_chunks);
        int vthreads = ((items + 1) / 2 + 31) / 32 * 32;
        vthreads = vthreads < 64 ? 64 : (vthreads > 256 ? 256 : vthreads);
        if (dtype == RDL_BF16)
            e = rdl_launch(rope_cache_vec_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(vthreads), 0, st, (__nv_bfloat16*)qkv, n_heads,
                           n_kv_heads, head_dim, rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, do_write,
                           (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, tables, table_width, page_size, ring_pages, seq_end);
        else
            e = rdl_launch(rope_cache_vec_kernel<float>, dim3(n_tokens), dim3(vthreads), 0, st, (float*)qkv, n_heads, n_kv_heads,
                           head_dim, rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, do_write, (float*)k_cache,
                           (float*)v_cache, tables, table_width, page_size, ring_pages, seq_end);
        RDL_CHECK_EX(e, "rope_cache");
        return 0;
    }
    dim3 grid(n_tokens, total_heads);
    const int threads = head_dim >= 256 ? 128 : (head_dim >= 64 ? 64 : 32);
    if (dtype == RDL_BF16)
        e = rdl_launch(rope_cache_kernel<__nv_bfloat16>, grid, dim3(threads), 0, st, (__nv_bfloat16*)qkv, n_heads, n_kv_heads, head_dim,
                       rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, do_write, (__nv_bfloat16*)k_cache,
                       (__nv_bfloat16*)v_cache, tables, table_width, page_size, ring_pages, seq_end);
    else
        e = rdl_launch(rope_cache_kernel<float>, grid, dim3(threads), 0, st, (float*)qkv, n_heads, n_kv_heads, head_dim,
                       rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, do_write, (float*)k_cache,
                       (float*)v_cache, tables, table_width, page_size, ring_pages, seq_end);
    RDL_CHECK_EX(e, "rope_cache");
    return 0;
}

// Rotation, a root-mean-square norm of every query and key head, and the cache write in one pass over packed
// rows with a stride of their own.  A warp takes a head: it rotates in float into its slice of shared memory,
// sums the squares in a fixed order (lane by lane, then across the warp), scales, and rounds once on the way
// back into the row and, for key heads, into the cache.  Value heads are copied to the cache as they are.
template <typename T>
__global__ void rope_norm_cache_kernel(T* __restrict__ rows, long long row_stride, int n_heads, int n_kv_heads, int head_dim,
                                       int rotary_dim, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                       const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, int do_rope,
                                       float norm_eps, int norm_dim, int do_write, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                       const int* __restrict__ tables, int table_width, int page_size, int ring_pages,
                                       const int* __restrict__ seq_end) {
    extern __shared__ float head_buf[];      // [warps][head_dim]
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    if (pos < 0) return;  // a padding row of a fixed-size batch
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    float* buf = head_buf + (size_t)warp * head_dim;
    bool write = do_write && n_kv_heads > 0;
    const int seq = tok_seq[t];
    // In a ring a later token of this step may land on the same row: only the last writer writes.
    if (write && (long long)pos + (long long)ring_pages * page_size < (long long)seq_end[seq]) write = false;
    const int r = pos % page_size;
    const int half = do_rope ? rotary_dim >> 1 : 0;
    const float* c = cos_t + (long long)pos * half;
    const float* s = sin_t + (long long)pos * half;
    const int total = n_heads + 2 * n_kv_heads;
    for (int head = warp; head < total; head += n_warps) {
        T* row = rows + (long long)t * row_stride + (long long)head * head_dim;
        const bool is_q = head < n_heads, is_v = head >= n_heads + n_kv_heads;
        T* dst = nullptr;
        if (write && !is_q) {
            const int kv_head = is_v ? head - n_heads - n_kv_heads : head - n_heads;
            dst = (is_v ? v_cache : k_cache) +
                  rdl_cache_offset(tables + (long long)seq * table_width, pos, page_size, ring_pages, n_kv_heads, kv_head, head_dim);
        }
        if (is_v) {
            if (dst)
                for (int i = lane; i < head_dim; i += 32) dst[rdl_cache_col<T>(r, i, head_dim)] = row[i];
            continue;
        }
        float ss = 0.f;
        for (int i = lane; i < half; i += 32) {
            const float x1 = to_float(row[i]), x2 = to_float(row[i + half]);
            const float cs = c[i], sn = s[i];
            const float lo = x1 * cs - x2 * sn, hi = x2 * cs + x1 * sn;
            buf[i] = lo;
            buf[i + half] = hi;
            ss = fmaf(lo, lo, ss);
            ss = fmaf(hi, hi, ss);
        }
        for (int i = 2 * half + lane; i < head_dim; i += 32) {
            const float x = to_float(row[i]);
            buf[i] = x;
            ss = fmaf(x, x, ss);
        }
        ss = warp_sum(ss);
        const float inv = norm_eps > 0.f ? 1.0f / sqrtf(ss / (float)norm_dim + norm_eps) : 1.0f;
        __syncwarp();
        for (int i = lane; i < head_dim; i += 32) {
            const T v = from_float<T>(buf[i] * inv);
            row[i] = v;
            if (dst) dst[rdl_cache_col<T>(r, i, head_dim)] = v;
        }
        __syncwarp();
    }
}

// The same with 16-byte accesses, for heads and rotated halves that are whole numbers of 16-byte chunks.  A head is taken
// by a group of LPH lanes (a power of two; 32 / LPH heads a warp at a time): a lane holds one rotated pair of chunks, or one
// chunk of the part that does not rotate, in registers; the squares are summed across the group in a fixed order; every
// value is loaded once and stored once.
template <typename T>
__global__ void __launch_bounds__(256) rope_norm_cache_vec_kernel(T* __restrict__ rows, long long row_stride, int n_heads, int n_kv_heads,
                                                                  int head_dim, int rotary_dim, const float* __restrict__ cos_t,
                                                                  const float* __restrict__ sin_t, const int* __restrict__ tok_seq,
                                                                  const int* __restrict__ tok_pos, int do_rope, float norm_eps, int norm_dim,
                                                                  int do_write, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                                  const int* __restrict__ tables, int table_width, int page_size,
                                                                  int ring_pages, const int* __restrict__ seq_end, int lph) {
    constexpr int N = Chunk<T>::N;
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    if (pos < 0) return;  // a padding row of a fixed-size batch
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const int per_warp = 32 / lph, sub = lane / lph, li = lane - sub * lph;
    const int chunks = head_dim / N, half = do_rope ? rotary_dim >> 1 : 0, hc = half / N;
    const int items = chunks - hc;                 // pairs, then single chunks
    bool write = do_write && n_kv_heads > 0;
    const int seq = tok_seq[t];
    // In a ring a later token of this step may land on the same row: only the last writer writes.
    if (write && (long long)pos + (long long)ring_pages * page_size < (long long)seq_end[seq]) write = false;
    const int r = pos % page_size;
    const int total = n_heads + 2 * n_kv_heads;
    for (int h0 = warp * per_warp; h0 < total; h0 += n_warps * per_warp) {     // the same trips for every lane of a warp
        const int head = h0 + sub;
        const bool live = head < total;
        const bool is_q = head < n_heads, is_v = head >= n_heads + n_kv_heads;
        T* row = rows + (long long)t * row_stride + (long long)(live ? head : 0) * head_dim;
        T* dst = nullptr;
        if (live && write && !is_q) {
            const int kv_head = is_v ? head - n_heads - n_kv_heads : head - n_heads;
            dst = (is_v ? v_cache : k_cache) +
                  rdl_cache_offset(tables + (long long)seq * table_width, pos, page_size, ring_pages, n_kv_heads, kv_head, head_dim);
        }
        if (live && is_v) {
            if (dst)
                for (int c = li; c < chunks; c += lph)
                    *reinterpret_cast<uint4*>(dst + rdl_swizzled_chunk(r, c, chunks) * N) = *reinterpret_cast<const uint4*>(row + c * N);
        }
        const bool mine = live && !is_v && li < items;
        const bool pair = mine && li < hc;
        const int c_lo = pair ? li : li + hc;      // the chunk this lane holds (and, for a pair, c_lo + hc)
        float a[N], b[N];
#pragma unroll
        for (int i = 0; i < N; ++i) a[i] = b[i] = 0.f;
        if (mine) Chunk<T>::load(row + c_lo * N, a);
        if (pair) {
            Chunk<T>::load(row + (c_lo + hc) * N, b);
            float cs[N], sn[N];
            const float4* cp = reinterpret_cast<const float4*>(cos_t + (long long)pos * half + c_lo * N);
            const float4* sp = reinterpret_cast<const float4*>(sin_t + (long long)pos * half + c_lo * N);
#pragma unroll
            for (int i = 0; i < N / 4; ++i) {
                const float4 cv = __ldg(cp + i), sv = __ldg(sp + i);
                cs[4 * i] = cv.x; cs[4 * i + 1] = cv.y; cs[4 * i + 2] = cv.z; cs[4 * i + 3] = cv.w;
                sn[4 * i] = sv.x; sn[4 * i + 1] = sv.y; sn[4 * i + 2] = sv.z; sn[4 * i + 3] = sv.w;
            }
#pragma unroll
            for (int i = 0; i < N; ++i) {
                const float lo = a[i] * cs[i] - b[i] * sn[i], hi = b[i] * cs[i] + a[i] * sn[i];
                a[i] = lo;
                b[i] = hi;
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < N; ++i) { ss = fmaf(a[i], a[i], ss); ss = fmaf(b[i], b[i], ss); }
        for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = norm_eps > 0.f ? 1.0f / sqrtf(ss / (float)norm_dim + norm_eps) : 1.0f;
        if (mine) {
#pragma unroll
            for (int i = 0; i < N; ++i) { a[i] *= inv; b[i] *= inv; }
            const uint4 pa = Chunk<T>::pack(a);
            *reinterpret_cast<uint4*>(row + c_lo * N) = pa;
            if (dst) *reinterpret_cast<uint4*>(dst + rdl_swizzled_chunk(r, c_lo, chunks) * N) = pa;
            if (pair) {
                const uint4 pb = Chunk<T>::pack(b);
                *reinterpret_cast<uint4*>(row + (c_lo + hc) * N) = pb;
                if (dst) *reinterpret_cast<uint4*>(dst + rdl_swizzled_chunk(r, c_lo + hc, chunks) * N) = pb;
            }
        }
    }
}

// A root-mean-square norm over the WHOLE query projection and over the WHOLE key projection of a token (all heads at
// once, one learned weight per column), then the rotation, then the cache write, in one pass over packed rows:
//     q <- R_pos(q / sqrt(sum(q^2) / q_count + eps) * wq),   k likewise with wk and k_count;   values are copied.
// q_count / k_count: the projections' true sizes (heads laid out with zero padding count their unpadded values).
// One block per token.  First the two sums of squares (lane by lane, across each warp, then the warps' parts in rising
// order: the order depends on the sizes alone), then a work item per rotated pair of pieces, per piece that does not
// rotate and per value piece; all in float, every value rounded once on the way back into the row and into the cache.
// VEC: pieces of 16 bytes (head_dim and rotary_dim / 2 whole numbers of them; weights and angles then come four at a time),
// else single values.
// Two other forms were measured on 2,048 tokens of 16 + 8 heads of 128 and not kept (this one, 256 threads: 23.4 us): a block
// per token with its pieces held in registers across the sums, 32.4 us, and a warp per token with its pieces in registers and
// the sums by shuffles, 49.9 us (33 us for 8 tokens): their unrolled bodies are long straight-line code that every warp runs once.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) rope_projnorm_cache_kernel(T* __restrict__ rows, long long row_stride, int n_heads, int n_kv_heads,
                                                                  int head_dim, int rotary_dim, const float* __restrict__ cos_t,
                                                                  const float* __restrict__ sin_t, const int* __restrict__ tok_seq,
                                                                  const int* __restrict__ tok_pos, int do_rope, const float* __restrict__ wq,
                                                                  const float* __restrict__ wk, float eps, float q_count, float k_count,
                                                                  int do_write, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                                  const int* __restrict__ tables, int table_width, int page_size,
                                                                  int ring_pages, const int* __restrict__ seq_end) {
    constexpr int N = VEC ? Chunk<T>::N : 1;
    __shared__ float part[2][8];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    if (pos < 0) return;  // a padding row of a fixed-size batch
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    T* row = rows + (long long)t * row_stride;
    const int qw = n_heads * head_dim, kw = n_kv_heads * head_dim;
    auto load = [](const T* p, float (&f)[N]) {
        if constexpr (VEC) Chunk<T>::load(p, f);
        else f[0] = to_float(*p);
    };
    auto store = [](T* p, const float (&f)[N]) {
        if constexpr (VEC) *reinterpret_cast<uint4*>(p) = Chunk<T>::pack(f);
        else *p = from_float<T>(f[0]);
    };
    auto table = [](const float* p, float (&f)[N]) {      // N weights or angles
        if constexpr (VEC) {
#pragma unroll
            for (int e = 0; e < N; e += 4) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(p + e));
                f[e] = v.x; f[e + 1] = v.y; f[e + 2] = v.z; f[e + 3] = v.w;
            }
        } else {
            f[0] = *p;
        }
    };
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x * N; i < qw + kw; i += blockDim.x * N) {
        float f[N];
        load(row + i, f);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < N; ++j) s = fmaf(f[j], f[j], s);
        if (i < qw) sq += s; else sk += s;
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if (lane == 0) { part[0][warp] = sq; part[1][warp] = sk; }
    __syncthreads();
    sq = sk = 0.f;
    for (int w = 0; w < n_warps; ++w) { sq += part[0][w]; sk += part[1][w]; }
    const float inv_q = 1.0f / sqrtf(sq / q_count + eps), inv_k = k_count > 0.f ? 1.0f / sqrtf(sk / k_count + eps) : 0.f;

    bool write = do_write && n_kv_heads > 0;
    const int seq = tok_seq[t];
    // In a ring a later token of this step may land on the same row: only the last writer writes.
    if (write && (long long)pos + (long long)ring_pages * page_size < (long long)seq_end[seq]) write = false;
    const int r = pos % page_size;
    const int half = do_rope ? rotary_dim >> 1 : 0;
    const int chunks = head_dim / N, hc = half / N;
    const int per_head = chunks - hc;                      // pairs, then pieces that do not rotate
    const int qk_items = (n_heads + n_kv_heads) * per_head;
    const int total = qk_items + (write ? n_kv_heads * chunks : 0);
    const int* page_list = tables + (long long)seq * table_width;
    for (int it = threadIdx.x; it < total; it += blockDim.x) {
        if (it >= qk_items) {                              // a piece of a value head, copied as it is
            const int v = it - qk_items, head = v / chunks, c = v - head * chunks;
            float f[N];
            load(row + qw + kw + head * head_dim + c * N, f);
            T* dst = v_cache + rdl_cache_offset(page_list, pos, page_size, ring_pages, n_kv_heads, head, head_dim);
            store(dst + (VEC ? rdl_swizzled_chunk(r, c, chunks) * N : rdl_cache_col<T>(r, c, head_dim)), f);
            continue;
        }
        const int head = it / per_head, j = it - head * per_head;
        const bool is_q = head < n_heads;
        const float inv = is_q ? inv_q : inv_k;
        const float* w = is_q ? wq + head * head_dim : wk + (head - n_heads) * head_dim;
        T* hrow = row + head * head_dim;
        T* dst = (write && !is_q) ? k_cache + rdl_cache_offset(page_list, pos, page_size, ring_pages, n_kv_heads, head - n_heads, head_dim) : nullptr;
        auto place = [&](int c) { return VEC ? rdl_swizzled_chunk(r, c, chunks) * N : rdl_cache_col<T>(r, c, head_dim); };
        if (j < hc) {
            const int i0 = j * N;
            float a[N], b[N], wa[N], wb[N], cs[N], sn[N];
            load(hrow + i0, a);
            load(hrow + i0 + half, b);
            table(w + i0, wa);
            table(w + i0 + half, wb);
            table(cos_t + (long long)pos * half + i0, cs);
            table(sin_t + (long long)pos * half + i0, sn);
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const float u = a[e] * inv * wa[e], v = b[e] * inv * wb[e];
                a[e] = u * cs[e] - v * sn[e];
                b[e] = v * cs[e] + u * sn[e];
            }
            store(hrow + i0, a);
            store(hrow + i0 + half, b);
            if (dst) { store(dst + place(j), a); store(dst + place(j + hc), b); }
        } else {
            const int c = j + hc, i0 = c * N;
            float a[N], wa[N];
            load(hrow + i0, a);
            table(w + i0, wa);
#pragma unroll
            for (int e = 0; e < N; ++e) a[e] = a[e] * inv * wa[e];
            store(hrow + i0, a);
            if (dst) store(dst + place(c), a);
        }
    }
}

extern "C" int rdl_rope_projnorm_cache(void* rows, long long row_stride, int dtype, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                       int rotary_dim, const float* cos_table, const float* sin_table, const int* tok_seq,
                                       const int* tok_pos, int do_rope, const float* wq, const float* wk, float eps, int q_count,
                                       int k_count, int do_write, void* k_cache, void* v_cache, const int* tables, int table_width,
                                       int page_size, int ring_pages, const int* seq_end, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "rope_projnorm_cache: bad dtype %d", dtype);
    RDL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads >= 0 && head_dim > 0 && head_dim <= 4096,
                "rope_projnorm_cache: bad sizes tokens=%d heads=%d kv_heads=%d head_dim=%d", n_tokens, n_heads, n_kv_heads, head_dim);
    RDL_REQUIRE(row_stride >= (long long)(n_heads + 2 * n_kv_heads) * head_dim, "rope_projnorm_cache: the row stride is below the heads' width");
    RDL_REQUIRE(!do_rope || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim && cos_table && sin_table),
                "rope_projnorm_cache: rotary_dim %d must be even and at most head_dim %d", rotary_dim, head_dim);
    RDL_REQUIRE(wq && (wk || n_kv_heads == 0) && eps > 0.f && q_count > 0 && q_count <= n_heads * head_dim &&
                    (n_kv_heads == 0 || (k_count > 0 && k_count <= n_kv_heads * head_dim)),
                "rope_projnorm_cache: the norms need weights, eps > 0 and the projections' true sizes");
    RDL_REQUIRE(tok_seq && tok_pos, "rope_projnorm_cache: missing batch description");
    RDL_REQUIRE(!do_write || n_kv_heads == 0 ||
                    (k_cache && v_cache && tables && seq_end && page_size > 0 && ring_pages > 0 && ring_pages <= table_width),
                "rope_projnorm_cache: cache write needs storage, page tables and lengths");
    if (n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int per_chunk = dtype == RDL_BF16 ? 8 : 4;
    const int half = do_rope ? rotary_dim / 2 : 0;
    const bool vec = head_dim % per_chunk == 0 && half % per_chunk == 0 && row_stride % per_chunk == 0 &&
                     (((uintptr_t)rows | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)wq | (uintptr_t)wk | (uintptr_t)cos_table |
                       (uintptr_t)sin_table) & 15) == 0;
    cudaError_t e;
    // bfloat16 steps of many tokens: small blocks, so that a multiprocessor holds many tokens (a block is a chain of a trip to
    // memory, a barrier and a second trip; 8,192 tokens of 16 + 8 heads of 128 took 99 us with 256 threads, 69 with 128, 65 with
    // 64).  Few tokens, and every 32-bit step (whose sums must not depend on the step's row count): 256 threads.
    const int threads = dtype == RDL_BF16 && n_tokens >= 256 ? 64 : 256;
#define RDL_PROJNORM(T, V)                                                                                                               \
    e = rdl_launch(rope_projnorm_cache_kernel<T, V>, dim3(n_tokens), dim3(threads), 0, st, (T*)rows, row_stride, n_heads, n_kv_heads, head_dim, \
                   rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, wq, wk, eps, (float)q_count, (float)k_count, do_write,   \
                   (T*)k_cache, (T*)v_cache, tables, table_width, page_size, ring_pages, seq_end)
    if (dtype == RDL_BF16) { if (vec) RDL_PROJNORM(__nv_bfloat16, true); else RDL_PROJNORM(__nv_bfloat16, false); }
    else { if (vec) RDL_PROJNORM(float, true); else RDL_PROJNORM(float, false); }
#undef RDL_PROJNORM
    RDL_CHECK_EX(e, "rope_projnorm_cache");
    return 0;
}

extern "C" int rdl_rope_norm_cache(void* rows, long long row_stride, int dtype, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                   int rotary_dim, const float* cos_table, const float* sin_table, const int* tok_seq,
                                   const int* tok_pos, int do_rope, float norm_eps, int norm_dim, int do_write, void* k_cache,
                                   void* v_cache, const int* tables, int table_width, int page_size, int ring_pages,
                                   const int* seq_end, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "rope_norm_cache: bad dtype %d", dtype);
    RDL_REQUIRE(n_tokens >= 0 && n_heads >= 0 && n_kv_heads >= 0 && n_heads + n_kv_heads > 0 && head_dim > 0 && head_dim <= 4096,
                "rope_norm_cache: bad sizes tokens=%d heads=%d kv_heads=%d head_dim=%d", n_tokens, n_heads, n_kv_heads, head_dim);
    RDL_REQUIRE(row_stride >= (long long)(n_heads + 2 * n_kv_heads) * head_dim, "rope_norm_cache: the row stride is below the heads' width");
    RDL_REQUIRE(!do_rope || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim && cos_table && sin_table),
                "rope_norm_cache: rotary_dim %d must be even and at most head_dim %d", rotary_dim, head_dim);
    RDL_REQUIRE(norm_eps <= 0.f || (norm_dim > 0 && norm_dim <= head_dim), "rope_norm_cache: norm_dim %d must lie in 1..head_dim", norm_dim);
    RDL_REQUIRE(tok_seq && tok_pos, "rope_norm_cache: missing batch description");
    RDL_REQUIRE(!do_write || n_kv_heads == 0 ||
                    (k_cache && v_cache && tables && seq_end && page_size > 0 && ring_pages > 0 && ring_pages <= table_width),
                "rope_norm_cache: cache write needs storage, page tables and lengths");
    if (n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    {
        const int per_chunk = dtype == RDL_BF16 ? 8 : 4;
        const int half = do_rope ? rotary_dim / 2 : 0;
        const bool aligned = (((uintptr_t)rows | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)cos_table | (uintptr_t)sin_table) & 15) == 0;
        const int items = head_dim % per_chunk == 0 && half % per_chunk == 0 ? head_dim / per_chunk - half / per_chunk : 0;
        if (aligned && items > 0 && items <= 32 && row_stride % per_chunk == 0) {
            int lph = 1;
            while (lph < items) lph *= 2;
            const int per_warp = 32 / lph, total = n_heads + 2 * n_kv_heads;
            int warps = (total + per_warp - 1) / per_warp;
            warps = warps > 8 ? 8 : warps;
            if (dtype == RDL_BF16)
                e = rdl_launch(rope_norm_cache_vec_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(warps * 32), 0, st, (__nv_bfloat16*)rows, row_stride,
                               n_heads, n_kv_heads, head_dim, rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, norm_eps, norm_dim,
                               do_write, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, tables, table_width, page_size, ring_pages, seq_end, lph);
            else
                e = rdl_launch(rope_norm_cache_vec_kernel<float>, dim3(n_tokens), dim3(warps * 32), 0, st, (float*)rows, row_stride, n_heads,
                               n_kv_heads, head_dim, rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, norm_eps, norm_dim, do_write,
                               (float*)k_cache, (float*)v_cache, tables, table_width, page_size, ring_pages, seq_end, lph);
            RDL_CHECK_EX(e, "rope_norm_cache");
            return 0;
        }
    }
    // a warp per head while a block's shared memory and thread count allow it: a head is three dependent steps
    // (load and rotate, sum, scale and store), so heads one after another in a warp are trips to memory one after another
    int warps = n_heads + 2 * n_kv_heads;
    if (warps > 16) warps = 16;
    while (warps > 1 && (size_t)warps * head_dim * sizeof(float) > 40 * 1024) warps /= 2;
    const size_t smem = (size_t)warps * head_dim * sizeof(float);
    if (dtype == RDL_BF16)
        e = rdl_launch(rope_norm_cache_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(warps * 32), smem, st, (__nv_bfloat16*)rows, row_stride,
                       n_heads, n_kv_heads, head_dim, rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, norm_eps, norm_dim,
                       do_write, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, tables, table_width, page_size, ring_pages, seq_end);
    else
        e = rdl_launch(rope_norm_cache_kernel<float>, dim3(n_tokens), dim3(warps * 32), smem, st, (float*)rows, row_stride, n_heads,
                       n_kv_heads, head_dim, rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, norm_eps, norm_dim, do_write,
                       (float*)k_cache, (float*)v_cache, tables, table_width, page_size, ring_pages, seq_end);
    RDL_CHECK_EX(e, "rope_norm_cache");
    return 0;
}
