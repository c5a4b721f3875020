// Decode attention of the latent-attention mixer (absorbed form) on tensor cores.
//
// One cached row [c | kr] per key serves every query head as key (all kv_rank + rot_dim values) and as value (its
// first kv_rank values).  A block takes one token, one group of 16 query heads and one run of keys (a split):
// the keys come into shared memory once, 64 at a time, and all 16 heads use them -
//     S[16 heads x 64 keys] = Q K^T            mma.sync m16n8k16, bfloat16 operands, float sums; warp w takes keys 8 w ..
//     online softmax in float (row maxima and sums exchanged between the eight warps through shared memory)
//     O[16 heads x kv_rank] += P V             warp w takes every eighth pair of 8-column tiles of the values
// Cache rows are copied as they lie (their 16-byte chunks XOR-swizzled by the row's place in its page), which is the
// layout ldmatrix reads without bank conflicts; Q and P are kept in shared memory in the same manner.
// A block holds one tile at a time (cp.async); two blocks share a multiprocessor (rows of up to 640 values leave room for
// both), so one computes while the other's copies travel.  With one split the block writes the heads' results itself; with more,
// each split leaves (max, sum, unnormalised O) in scratch and a second kernel merges them in a fixed order.
// Sizes: kv_rank + rot_dim a multiple of 16 up to 640, kv_rank a multiple of 16 up to 512, pages of a multiple of 8
// positions; any number of heads.
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

constexpr int LD_TILE = 64, LD_WARPS = 8, LD_THREADS = LD_WARPS * 32, LD_HEADS = 16;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// byte offset of element i of a swizzled row: 16-byte chunk c lies at c ^ (key & 7) inside complete groups of eight
__device__ __forceinline__ int swz(int key, int i, int chunks) {
    const int c = i >> 3;
    return (rdl_swizzled_chunk(key, c, chunks) << 4) + ((i & 7) << 1);
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

struct LatentDecodeArgs {
    const __nv_bfloat16* q; long long q_stride;      // [tokens][heads * width]
    const __nv_bfloat16* cache;                      // [pages][1][page_size][width]
    __nv_bfloat16* out; long long out_stride;        // [tokens][heads * width]: the first kv_rank values of each head are written
    const int* tok_seq; const int* tok_pos; const int* tables;
    int table_width, page_size, ring_pages;
    int n_heads, width, kv_rank, window;
    float scale_log2;                                // score scale * log2(e)
    int tiles_per_split, n_splits;
    float* partial;                                  // [tokens][head groups * 16][splits][kv_rank + 2] (splits > 1)
    const float* sinks;                              // optional [heads]: a logit that joins the denominator once, unscaled
};

// byte offset of 16-byte chunk c of a row whose chunk count is a multiple of 8 (every group of eight is swizzled)
__device__ __forceinline__ int swz_chunk(int key7, int c) { return (c ^ key7) << 4; }

// NP: pairs of 8-column value tiles a warp accumulates (kv_rank <= 128 NP).  FULL: a row is a whole number of groups of
// eight chunks (128 bytes), so every chunk is swizzled and its place is one XOR away.
template <int NP, bool FULL>
__global__ void __launch_bounds__(LD_THREADS, 2) latent_decode_kernel(LatentDecodeArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int width = a.width, chunks = width >> 3, row_bytes = width * 2;
    unsigned char* q_s = smem;                                    // [16][width]
    unsigned char* p_s = q_s + LD_HEADS * row_bytes;              // [16][64]
    float* wmax = (float*)(p_s + LD_HEADS * LD_TILE * 2);         // [8][16]
    float* wsum = wmax + LD_WARPS * LD_HEADS;                     // [8][16]
    long long* key_off = (long long*)(wsum + LD_WARPS * LD_HEADS);   // [64] where each key's row starts in the cache; -1: not read
    unsigned char* k_s = (unsigned char*)(key_off + LD_TILE);        // [64][width]: one tile; a second block on the multiprocessor computes while this one's copies travel

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x, hg = blockIdx.y, t = blockIdx.z;
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int p = a.tok_pos[t];
    if (p < 0) return;                                            // a padding row of a fixed-size batch
    const int seq = a.tok_seq[t];
    const int* table = a.tables + (long long)seq * a.table_width;
    const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
    const int first_tile = lo / LD_TILE + split * a.tiles_per_split;
    const int last_tile = min(p / LD_TILE, first_tile + a.tiles_per_split - 1);
    const int n_tiles = last_tile - first_tile + 1;               // may be <= 0: a split beyond this token's keys

    // A tile's copies: 64 threads look the rows up in the page list, then every warp copies rows as they lie (their
    // chunks are swizzled already), a lane a 16-byte chunk; rows outside the token's keys are zero.
    auto load_tile = [&](int tile) {
        unsigned char* dst = k_s;
        const int pos0 = tile * LD_TILE;
        if (threadIdx.x < LD_TILE) {
            const int pos = pos0 + threadIdx.x;
            key_off[threadIdx.x] = (pos >= lo && pos <= p) ? rdl_cache_offset(table, pos, a.page_size, a.ring_pages, 1, 0, width) : -1;
        }
        __syncthreads();
        for (int key = warp; key < LD_TILE; key += LD_WARPS) {
            const long long off = key_off[key];
            unsigned char* d = dst + key * row_bytes + (lane << 4);
            if (off >= 0) {                                        // uniform over the warp
                const unsigned char* src = (const unsigned char*)(a.cache + off) + (lane << 4);
                uint32_t da = smem_addr(d);
                for (int c = lane; c < chunks; c += 32, da += 512, src += 512) cp_async16(da, src);
            } else {
                for (int c = lane; c < chunks; c += 32, d += 512) *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    const int g = lane >> 2, qd = lane & 3;                       // accumulator rows g and g + 8, columns 2 qd, 2 qd + 1
    float o[NP][2][4];
#pragma unroll
    for (int i = 0; i < NP; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[i][j][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int n_pairs = a.kv_rank >> 4;                           // pairs of value tiles in all

    if (n_tiles > 0) load_tile(first_tile);
    // queries of this head group, swizzled by head row; heads beyond the last are zero (the first tile's copies are on
    // their way meanwhile)
    for (int i = threadIdx.x; i < LD_HEADS * chunks; i += LD_THREADS) {
        const int h = i / chunks, c = i - h * chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (hg * LD_HEADS + h < a.n_heads)
            v = *reinterpret_cast<const uint4*>(a.q + (long long)t * a.q_stride + (long long)(hg * LD_HEADS + h) * width + c * 8);
        *reinterpret_cast<uint4*>(q_s + h * row_bytes + (rdl_swizzled_chunk(h, c, chunks) << 4)) = v;
    }

    for (int it = 0; it < n_tiles; ++it) {
        if (it > 0) load_tile(first_tile + it);                   // the sync that ended the tile before has freed the buffer
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                          // the tile (and, the first time, Q) is in shared memory
        const unsigned char* kt = k_s;
        const int pos0 = (first_tile + it) * LD_TILE;
        // ---- S = Q K^T for this warp's 8 keys; one load of K fragments serves two steps of 16 along the row ----
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const int a_row = lane & 15, a_k = (lane >> 4) << 3;
            const int b_key = warp * 8 + (lane & 7), b_k = (lane >> 3) << 3;
            const int b_sw = (pos0 + b_key) % a.page_size;        // the row's place in its page: what its chunks were swizzled by
            const uint32_t q_row = smem_addr(q_s + a_row * row_bytes), k_row = smem_addr(kt + b_key * row_bytes);
            float s2[4] = {0.f, 0.f, 0.f, 0.f};                   // a second chain of sums: the steps alternate between the two
            if (FULL) {
                // chunk indices of this lane's fragment rows at k0 = 0; a step of 32 values is four chunks further
                const int qc = a_k >> 3, kc = b_k >> 3, q7 = a_row & 7, k7 = b_sw & 7;
#pragma unroll 2
                for (int c0 = 0; c0 < chunks; c0 += 4) {
                    uint32_t af[4], af2[4], bf[4];
                    ldsm_x4(k_row + swz_chunk(k7, c0 + kc), bf);
                    ldsm_x4(q_row + swz_chunk(q7, c0 + qc), af);
                    ldsm_x4(q_row + swz_chunk(q7, c0 + 2 + qc), af2);
                    mma16816(s, af, bf[0], bf[1]);
                    mma16816(s2, af2, bf[2], bf[3]);
                }
            } else {
#pragma unroll 2
                for (int k0 = 0; k0 < width; k0 += 32) {
                    uint32_t af[4], af2[4], bf[4];
                    const bool two = k0 + 16 < width;
                    // beyond the row's end (its last step of 16) the second half of the load reads the next row and is not used
                    ldsm_x4(k_row + swz(b_sw, k0 + b_k, chunks), bf);
                    ldsm_x4(q_row + swz(a_row, k0 + a_k, chunks), af);
                    if (two) ldsm_x4(q_row + swz(a_row, k0 + 16 + a_k, chunks), af2);
                    mma16816(s, af, bf[0], bf[1]);
                    if (two) mma16816(s2, af2, bf[2], bf[3]);
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) s[e] += s2[e];
        }
        // ---- mask, row maxima over the warps ----
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int pos = pos0 + warp * 8 + 2 * qd + (e & 1);
            const float v = (pos >= lo && pos <= p) ? s[e] * a.scale_log2 : -INFINITY;
            s[e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        }
        if (qd == 0) { wmax[warp * LD_HEADS + g] = mx[0]; wmax[warp * LD_HEADS + g + 8] = mx[1]; }
        __syncthreads();
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = g + 8 * r;
            float tm = wmax[row];
#pragma unroll
            for (int w = 1; w < LD_WARPS; ++w) tm = fmaxf(tm, wmax[w * LD_HEADS + row]);
            const float m_new = fmaxf(m_run[r], tm);
            m_use[r] = m_new == -INFINITY ? 0.f : m_new;
            corr[r] = exp2f(m_run[r] - m_use[r]);                 // 0 while nothing has been seen
            m_run[r] = m_new;
        }
        // ---- P = 2^(S - m), row sums, P into shared memory as bfloat16 ----
        float sm[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float p0 = exp2f(s[2 * r] - m_use[r]), p1 = exp2f(s[2 * r + 1] - m_use[r]);
            const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
            // the sums are those of the rounded weights, which is what multiplies the values
            sm[r] = __bfloat162float(pb.x) + __bfloat162float(pb.y);
            const int row = g + 8 * r, col = warp * 8 + 2 * qd;
            *reinterpret_cast<__nv_bfloat162*>(p_s + row * (LD_TILE * 2) + swz_chunk(row & 7, col >> 3) + ((col & 7) << 1)) = pb;
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            sm[r] += __shfl_xor_sync(0xffffffffu, sm[r], 1);
            sm[r] += __shfl_xor_sync(0xffffffffu, sm[r], 2);
        }
        if (qd == 0) { wsum[warp * LD_HEADS + g] = sm[0]; wsum[warp * LD_HEADS + g + 8] = sm[1]; }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = g + 8 * r;
            float ts = 0.f;
#pragma unroll
            for (int w = 0; w < LD_WARPS; ++w) ts += wsum[w * LD_HEADS + row];      // a fixed order
            l_run[r] = l_run[r] * corr[r] + ts;
        }
        // ---- O = O * corr + P V for this warp's value tiles ----
#pragma unroll
        for (int i = 0; i < NP; ++i)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                o[i][j][0] *= corr[0]; o[i][j][1] *= corr[0];
                o[i][j][2] *= corr[1]; o[i][j][3] *= corr[1];
            }
        {
            const int a_row = lane & 15, a_k = (lane >> 4) << 3;
            const int v_key = lane & 15, v_n = (lane >> 4) << 3;
#pragma unroll
            for (int kk = 0; kk < LD_TILE; kk += 16) {
                uint32_t pf[4];
                ldsm_x4(smem_addr(p_s + a_row * (LD_TILE * 2)) + swz_chunk(a_row & 7, (kk + a_k) >> 3), pf);
                const int key = kk + v_key;
                const int sw = (pos0 + key) % a.page_size;
                const uint32_t v_row = smem_addr(kt + key * row_bytes);
#pragma unroll
                for (int i = 0; i < NP; ++i) {
                    const int pair = warp + LD_WARPS * i;
                    if (pair < n_pairs) {
                        uint32_t vf[4];
                        ldsm_x4_t(v_row + (FULL ? swz_chunk(sw & 7, pair * 2 + (v_n >> 3)) : swz(sw, pair * 16 + v_n, chunks)), vf);
                        mma16816(o[i][0], pf, vf[0], vf[1]);
                        mma16816(o[i][1], pf, vf[2], vf[3]);
                    }
                }
            }
        }
        __syncthreads();                                          // the tile, P and the exchange arrays are free again
    }

    // ---- results ----
    const int r_dim = a.kv_rank;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int head = hg * LD_HEADS + g + 8 * r;
        if (head >= a.n_heads) continue;
        if (a.n_splits == 1) {
            float l = l_run[r];
            if (a.sinks) {      // base-2 domain, like m_run; with no key seen the sink alone fills the denominator and O is zero
                const float sk = a.sinks[head] * 1.4426950408889634f;
                l = m_run[r] == -INFINITY ? 1.0f : l + exp2f(sk - m_run[r]);
            }
            const float inv = 1.0f / l;
            __nv_bfloat16* dst = a.out + (long long)t * a.out_stride + (long long)head * width;
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                const int pair = warp + LD_WARPS * i;
                if (pair >= n_pairs) continue;
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    *reinterpret_cast<__nv_bfloat162*>(dst + pair * 16 + j * 8 + 2 * qd) =
                        __floats2bfloat162_rn(o[i][j][2 * r] * inv, o[i][j][2 * r + 1] * inv);
            }
        } else {
            float* dst = a.partial + (((long long)t * gridDim.y * LD_HEADS + (hg * LD_HEADS + g + 8 * r)) * a.n_splits + split) * (r_dim + 2);
            if (warp == 0 && qd == 0) { dst[r_dim] = m_run[r]; dst[r_dim + 1] = l_run[r]; }
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                const int pair = warp + LD_WARPS * i;
                if (pair >= n_pairs) continue;
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    *reinterpret_cast<float2*>(dst + pair * 16 + j * 8 + 2 * qd) = make_float2(o[i][j][2 * r], o[i][j][2 * r + 1]);
            }
        }
    }
}

// out[t, h, :kv_rank] = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), splits in rising order.  The splits' factors
// are formed once (shared memory); the sums then read their terms with all loads in flight.
constexpr int LD_MAX_SPLITS = 64;

__global__ void __launch_bounds__(128) latent_decode_merge_kernel(LatentDecodeArgs a, int head_rows) {
    __shared__ float factor[LD_MAX_SPLITS];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.y, head = blockIdx.x;
    if (a.tok_pos[t] < 0) return;
    const int r_dim = a.kv_rank, stride = r_dim + 2;
    const float* base = a.partial + (((long long)t * head_rows + head) * a.n_splits) * stride;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float m[2], l[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int s = lane + 32 * i;
            m[i] = s < a.n_splits ? base[(long long)s * stride + r_dim] : -INFINITY;
            l[i] = s < a.n_splits ? base[(long long)s * stride + r_dim + 1] : 0.f;
        }
        const float M = warp_max(fmaxf(m[0], m[1]));
        float f[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) f[i] = m[i] == -INFINITY ? 0.f : exp2f(m[i] - M);
        // the sum over the splits in rising order, by one lane from shared memory (a shuffle tree would order it otherwise)
        factor[lane] = l[0] * f[0];
        factor[lane + 32] = l[1] * f[1];
        __syncwarp();
        float L = 0.f;
        if (lane == 0)
            for (int s = 0; s < a.n_splits; ++s) L += factor[s];
        if (lane == 0 && a.sinks) L = M == -INFINITY ? 1.0f : L + exp2f(a.sinks[head] * 1.4426950408889634f - M);
        L = __shfl_sync(0xffffffffu, L, 0);
        __syncwarp();
        factor[lane] = f[0] / L;
        factor[lane + 32] = f[1] / L;
    }
    __syncthreads();
    __nv_bfloat16* dst = a.out + (long long)t * a.out_stride + (long long)head * a.width;
    for (int i = threadIdx.x; i < r_dim; i += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < a.n_splits; ++s) acc = fmaf(base[(long long)s * stride + i], factor[s], acc);
        dst[i] = __float2bfloat16_rn(acc);
    }
}

template <int NP, bool FULL>
int launch_latent_decode_form(const LatentDecodeArgs& a, dim3 grid, size_t smem, cudaStream_t st) {
    static bool opted = false;
    if (!opted) {
        RDL_CUDA(cudaFuncSetAttribute(latent_decode_kernel<NP, FULL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024), "latent_decode");
        opted = true;
    }
    RDL_CHECK_EX(rdl_launch(latent_decode_kernel<NP, FULL>, grid, dim3(LD_THREADS), smem, st, a), "latent_decode");
    return 0;
}

template <int NP>
int launch_latent_decode(const LatentDecodeArgs& a, dim3 grid, size_t smem, cudaStream_t st) {
    // rows of a multiple of 64 values: every chunk swizzled, and a step of 32 values never leaves the row
    return a.width % 64 == 0 ? launch_latent_decode_form<NP, true>(a, grid, smem, st) : launch_latent_decode_form<NP, false>(a, grid, smem, st);
}

}  // namespace

extern "C" long long rdl_latent_decode_scratch_bytes(int n_tokens, int n_heads, int kv_rank, int n_splits) {
    if (n_splits <= 1) return 0;
    const long long head_rows = (long long)((n_heads + LD_HEADS - 1) / LD_HEADS) * LD_HEADS;
    return (long long)n_tokens * head_rows * n_splits * (kv_rank + 2) * (long long)sizeof(float);
}

// q: [tokens][heads * width] rows of the absorbed form; out: the same shape, the first kv_rank values of every head written.
// max_keys: the longest run of keys any token of the batch reads; n_splits: blocks a token's keys are shared between
// (scratch of rdl_latent_decode_scratch_bytes when > 1).
extern "C" int rdl_latent_decode(void* out, long long out_stride, const void* q, long long q_stride, const void* cache, const int* tables,
                                 int table_width, int page_size, int ring_pages, const int* tok_seq, const int* tok_pos, int n_tokens,
                                 int n_heads, int width, int kv_rank, float score_scale, int window, int max_keys, int n_splits,
                                 void* scratch, long long scratch_bytes, const float* sinks, void* stream) {
    RDL_REQUIRE(out && q && cache && tables && tok_seq && tok_pos, "latent_decode: missing operand");
    RDL_REQUIRE(width % 16 == 0 && width <= 640 && kv_rank % 16 == 0 && kv_rank > 0 && kv_rank <= 512 && kv_rank <= width,
                "latent_decode: rows of %d values with %d latent values are not taken (multiples of 16 up to 640 and 512)", width, kv_rank);
    RDL_REQUIRE(page_size > 0 && page_size % 8 == 0 && ring_pages > 0 && ring_pages <= table_width, "latent_decode: bad paging (page_size %d)", page_size);
    RDL_REQUIRE(n_heads > 0 && window >= 0 && max_keys > 0 && n_splits >= 1, "latent_decode: bad sizes");
    RDL_REQUIRE(((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache) % 16 == 0 && q_stride % 8 == 0 && out_stride % 8 == 0, "latent_decode: rows must start on 16-byte boundaries");
    if (n_tokens == 0) return 0;
    RDL_REQUIRE(n_tokens <= 65535, "latent_decode: %d tokens exceed the grid limit", n_tokens);
    const int groups = (n_heads + LD_HEADS - 1) / LD_HEADS;
    const int tiles = (max_keys + LD_TILE - 1) / LD_TILE + 1;     // a run of max_keys positions can straddle one more tile
    if (n_splits > tiles) n_splits = tiles;
    if (n_splits > LD_MAX_SPLITS) n_splits = LD_MAX_SPLITS;
    RDL_REQUIRE(scratch_bytes >= rdl_latent_decode_scratch_bytes(n_tokens, n_heads, kv_rank, n_splits) && (n_splits == 1 || scratch),
                "latent_decode: scratch too small");
    LatentDecodeArgs a{(const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, out_stride, tok_seq, tok_pos, tables,
                       table_width, page_size, ring_pages, n_heads, width, kv_rank, window, score_scale * 1.4426950408889634f,
                       (tiles + n_splits - 1) / n_splits, n_splits, (float*)scratch, sinks};
    const size_t smem = (size_t)LD_HEADS * width * 2 + LD_HEADS * LD_TILE * 2 + 2 * LD_WARPS * LD_HEADS * sizeof(float) + LD_TILE * sizeof(long long) +
                        (size_t)LD_TILE * width * 2 + 64;          // 64: a fragment load may reach past the last row's end
    const dim3 grid(n_splits, groups, n_tokens);
    cudaStream_t st = (cudaStream_t)stream;
    int e;
    if (kv_rank <= 128) e = launch_latent_decode<1>(a, grid, smem, st);
    else if (kv_rank <= 256) e = launch_latent_decode<2>(a, grid, smem, st);
    else e = launch_latent_decode<4>(a, grid, smem, st);
    if (e) return e;
    if (n_splits > 1)
        RDL_CHECK_EX(rdl_launch(latent_decode_merge_kernel, dim3(n_heads, n_tokens), dim3(128), 0, st, a, groups * LD_HEADS), "latent_decode_merge");
    return 0;
}
