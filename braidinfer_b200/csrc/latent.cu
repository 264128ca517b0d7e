// Latent attention: keys and values of all heads live in one low-rank vector per token.
//
// Per token the cache keeps c (kv_rank numbers, an RMS-normed down-projection of the layer's input) and
// one rotated key part kr (rot_dim numbers) shared by all heads: D = kv_rank + rot_dim numbers in all.
// Head h's unrotated key is Wuk_h c and its value Wuv_h c.  Because the score is linear in the key,
//     q_u . (Wuk_h c) = (Wuk_h^T q_u) . c,
// a query head is first carried into the latent space (q~ = [Wuk_h^T q_u ; q_r], D numbers) and attention
// then runs as multi-query attention over the cached rows themselves: key = the whole row, value = its
// first kv_rank numbers.  The head's output is Wuv_h (sum_j p_j c_j).  The cache is never expanded.
//
// This file holds the plain kernels (float32 run, and the twin that the tensor-core kernels are tested
// against): the row preparation (norm of c, rotation of kr and of the queries' rotated parts, cache
// write), a per-head matrix product, and one-warp-per-(token, head) attention over the latent cache.
// Norm, angles, scores, softmax and accumulation are float32.
#include "common.cuh"
#include "mma_tile.cuh"

// ------------------------------------------------------------------ row preparation
struct LatentPrepArgs {
    const void* proj;         // [rows, ld]: queries at column 0 (heads x (dim + rot)), then c (rank), then kr (rot)
    long long ld;
    int q_cols;               // heads * (dim + rot): where c starts
    const void* norm_w;       // [rank]
    const float* inv_freq;    // [rot_pairs]
    const int* positions;     // [rows]
    const int* token_seq;     // [rows] or -1
    const int* page_table;    // [n_seqs, table_cols]
    void* cache;              // [pages][page_size][rank + rot], or null (no write)
    void* q_lat;              // [rows, heads, rank + rot]: the rotated parts are written at [.., rank:]
    int rows, heads, dim, rot, rank, rot_dims;     // rot_dims <= rot: the first rot_dims of the rotated part turn
    int page_size, table_cols, num_pages;
    float eps;
    int* error_flag;
    int adjacent;             // pairs are (2p, 2p + 1) instead of (p, p + rot_dims/2)
};

template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(LatentPrepArgs a) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int row = blockIdx.x;
    const int seq = a.token_seq[row];
    const int pos = seq < 0 ? 0 : a.positions[row];
    const int D = a.rank + a.rot;
    const T* src = (const T*)a.proj + (size_t)row * a.ld;
    const T* cin = src + a.q_cols;
    const T* kin = cin + a.rank;
    T* dst = nullptr;
    if (seq >= 0 && a.cache) {
        const int block = pos / a.page_size, off = pos - block * a.page_size;
        int page = (block < a.table_cols) ? a.page_table[(size_t)seq * a.table_cols + block] : -1;
        if (page < 0 || page >= a.num_pages) {
            if (threadIdx.x == 0) atomicExch(a.error_flag, 1);
        } else {
            dst = (T*)a.cache + ((size_t)page * a.page_size + off) * D;
        }
    }
    // c = x / sqrt(mean(x^2) + eps) * w  (only where there is a cache to write: a layer that reads another layer's
    // latent has no c and no kr in its rows)
    float ss = 0.f;
    if (a.cache) {
        for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
            const float v = to_f32(cin[i]);
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, red);
    }
    const float scale = 1.f / sqrtf(ss / (float)a.rank + a.eps);
    if (dst) {
        const T* w = (const T*)a.norm_w;
        for (int i = threadIdx.x; i < a.rank; i += blockDim.x) dst[i] = from_f32<T>(to_f32(cin[i]) * scale * to_f32(w[i]));
    }
    // rotation: element i pairs with i + rot_dims/2 (or, `adjacent`, 2i with 2i + 1); vector 0 is the shared key
    // part, 1.. are the heads' queries
    const int half = a.rot_dims / 2;
    const int per = half + (a.rot - a.rot_dims);           // work items a vector: pairs, then untouched elements
    for (int e = threadIdx.x; e < (a.heads + 1) * per; e += blockDim.x) {
        const int v = e / per, p = e - v * per;
        const T* in = (v == 0) ? kin : src + (size_t)(v - 1) * (a.dim + a.rot) + a.dim;
        T* out = (v == 0) ? (dst ? dst + a.rank : nullptr) : (T*)a.q_lat + ((size_t)row * a.heads + (v - 1)) * D + a.rank;
        if (!out) continue;
        if (p < half) {
            float sn, cs;
            sincosf((float)pos * a.inv_freq[p], &sn, &cs);
            const int i0 = a.adjacent ? 2 * p : p, i1 = a.adjacent ? 2 * p + 1 : p + half;
            const float x0 = to_f32(in[i0]), x1 = to_f32(in[i1]);
            out[i0] = from_f32<T>(x0 * cs - x1 * sn);
            out[i1] = from_f32<T>(x1 * cs + x0 * sn);
        } else {
            const int i = a.rot_dims + (p - half);
            out[i] = in[i];
        }
    }
}

extern "C" int braid_latent_prep(const void* proj, long long ld, int q_cols, const void* norm_w, const float* inv_freq,
                                 const int* positions, const int* token_seq, const int* page_table, void* cache,
                                 void* q_lat, int dtype, int rows, int heads, int dim, int rot, int rank, int rot_dims,
                                 int page_size, int table_cols, int num_pages, float eps, int adjacent, int* error_flag, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (heads <= 0 || dim < 0 || rot < 0 || rank <= 0) BRAID_REFUSE("latent_prep: heads=%d dim=%d rot=%d rank=%d", heads, dim, rot, rank);
    if (rot_dims < 0 || rot_dims > rot || rot_dims % 2) BRAID_REFUSE("latent_prep: %d rotated dimensions must be even and within %d", rot_dims, rot);
    if (!error_flag) BRAID_REFUSE("latent_prep: error_flag is required");
    if (cache && (!page_table || table_cols <= 0 || num_pages <= 0 || page_size <= 0)) BRAID_REFUSE("latent_prep: the cache has no pages");
    LatentPrepArgs a{proj, ld, q_cols, norm_w, inv_freq, positions, token_seq, page_table, cache, q_lat,
                     rows, heads, dim, rot, rank, rot_dims, page_size, table_cols, num_pages, eps, error_flag, adjacent};
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32) braid_launch(latent_prep_kernel<float>, dim3(rows), dim3(128), 0, s, a);
    else if (dtype == BRAID_BF16) braid_launch(latent_prep_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, s, a);
    else BRAID_REFUSE("latent_prep: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ per-head matrix product
// out[n, h, j] = sum_k x[n, h, k] * w[h, j, k]   (w: [heads, J, K], each head's matrix [out, in])
// x[n, h, k] lies at x + n*ldx + h*hsx + k, out[n, h, j] at out + n*ldo + h*hso + j.
// With `gate` the result is multiplied by mult * sigmoid(gate[n*ldg + h]) (one gate a token and head).
// float32 FMA in a fixed order along k.
#define HG_BM 64
#define HG_BN 64
#define HG_BK 16

template <typename T>
__global__ void __launch_bounds__(256)
gemm_heads_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out, const T* __restrict__ gate,
                  int n_rows, int J, int K, long long ldx, long long hsx, long long ldo, long long hso,
                  long long ldg, float mult) {
    pdl_trigger();
    pdl_wait();
    __shared__ float xs[HG_BK][HG_BN + 4];
    __shared__ float ws[HG_BK][HG_BM + 4];
    const int h = blockIdx.z;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int n0 = blockIdx.y * HG_BN, m0 = blockIdx.x * HG_BM;
    const T* xh = x + (size_t)h * hsx;
    const T* wh = w + (size_t)h * J * K;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HG_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = threadIdx.x + i * 256;
            const int r = e >> 4, c = e & 15;
            const int k = k0 + c;
            const int n = n0 + r, m = m0 + r;
            xs[c][r] = (n < n_rows && k < K) ? to_f32(xh[(size_t)n * ldx + k]) : 0.f;
            ws[c][r] = (m < J && k < K) ? to_f32(wh[(size_t)m * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HG_BK; ++kk) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int n = n0 + ty * 4 + i;
        if (n >= n_rows) continue;
        float g = 1.f;
        if (gate) g = mult / (1.f + expf(-to_f32(gate[(size_t)n * ldg + h])));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + tx * 4 + j;
            if (m >= J) continue;
            out[(size_t)n * ldo + (size_t)h * hso + m] = from_f32<T>(acc[i][j] * g);
        }
    }
}

extern "C" int braid_gemm_heads(const void* x, const void* w, void* out, const void* gate, int dtype,
                                int n_rows, int heads, int J, int K, long long ldx, long long hsx,
                                long long ldo, long long hso, long long ldg, float mult, void* stream) {
    if (n_rows <= 0 || heads <= 0 || J <= 0) return BRAID_OK;
    if (K <= 0) BRAID_REFUSE("gemm_heads: k=%d must be positive", K);
    dim3 grid((J + HG_BM - 1) / HG_BM, (n_rows + HG_BN - 1) / HG_BN, heads);
    if (grid.y > 65535 || grid.z > 65535) BRAID_REFUSE("gemm_heads: %d rows x %d heads exceed the grid limit", n_rows, heads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32)
        braid_launch(gemm_heads_kernel<float>, grid, dim3(256), 0, s, (const float*)x, (const float*)w, (float*)out,
                     (const float*)gate, n_rows, J, K, ldx, hsx, ldo, hso, ldg, mult);
    else if (dtype == BRAID_BF16)
        braid_launch(gemm_heads_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (const __nv_bfloat16*)x,
                     (const __nv_bfloat16*)w, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate, n_rows, J, K, ldx, hsx,
                     ldo, hso, ldg, mult);
    else BRAID_REFUSE("gemm_heads: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

// The same product in bfloat16 on the tensor cores (mma_tile.cuh): BM tokens x 64 outputs of one head a CTA.
template <int BM>
__global__ void __launch_bounds__(128)
gemm_heads_mma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                      const __nv_bfloat16* __restrict__ gate, int n_rows, int J, int K, long long ldx, long long hsx,
                      long long ldo, long long hso, long long ldg, float mult) {
    using Tile = MmaTile<BM, 64, (BM >= 64 ? 2 : 1), (BM >= 64 ? 2 : 4), 1>;
    extern __shared__ __align__(16) unsigned char hg_smem[];
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.z, n0 = blockIdx.y * BM, m0 = blockIdx.x * 64;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int ACH = BM * 4 / 128 > 0 ? BM * 4 / 128 : 1;
    const __nv_bfloat16* a_rows[ACH];
    const __nv_bfloat16* b_rows[1][2];
#pragma unroll
    for (int i = 0; i < ACH; ++i) {
        const int r = (tid + i * 128) >> 2;
        a_rows[i] = (r < BM && n0 + r < n_rows) ? x + (size_t)(n0 + r) * ldx + (size_t)h * hsx : nullptr;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = m0 + ((tid + i * 128) >> 2);
        b_rows[0][i] = m < J ? w + ((size_t)h * J + m) * K : nullptr;
    }
    float acc[1][Tile::MI][Tile::NI][4];
    Tile::run(acc, (__nv_bfloat16*)hg_smem, a_rows, b_rows, K, w);
    const int wm0 = (warp / (BM >= 64 ? 2 : 4)) * (BM / (BM >= 64 ? 2 : 1)), wn0 = (warp % (BM >= 64 ? 2 : 4)) * (64 / (BM >= 64 ? 2 : 4));
    const bool pairs_ok = ((ldo | hso) & 1) == 0;
#pragma unroll
    for (int mi = 0; mi < Tile::MI; ++mi)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int n = n0 + wm0 + mi * 16 + (lane >> 2) + half * 8;
            if (n >= n_rows) continue;
            float g = 1.f;
            if (gate) g = mult / (1.f + expf(-__bfloat162float(gate[(size_t)n * ldg + h])));
            __nv_bfloat16* orow = out + (size_t)n * ldo + (size_t)h * hso;
#pragma unroll
            for (int ni = 0; ni < Tile::NI; ++ni) {
                const int col = m0 + wn0 + ni * 8 + 2 * (lane & 3);
                const float v0 = acc[0][mi][ni][half * 2] * g, v1 = acc[0][mi][ni][half * 2 + 1] * g;
                if (pairs_ok && col + 1 < J) *reinterpret_cast<__nv_bfloat162*>(orow + col) = __floats2bfloat162_rn(v0, v1);
                else {
                    if (col < J) orow[col] = __float2bfloat16_rn(v0);
                    if (col + 1 < J) orow[col + 1] = __float2bfloat16_rn(v1);
                }
            }
        }
}

extern "C" int braid_gemm_heads_mma(const void* x, const void* w, void* out, const void* gate, int n_rows, int heads,
                                    int J, int K, long long ldx, long long hsx, long long ldo, long long hso,
                                    long long ldg, float mult, void* stream) {
    if (n_rows <= 0 || heads <= 0 || J <= 0) return BRAID_OK;
    if (K <= 0 || K % 8 || ldx % 8 || hsx % 8) BRAID_REFUSE("gemm_heads_mma: k=%d and the strides %lld, %lld must be multiples of 8", K, ldx, hsx);
    if (((uintptr_t)x | (uintptr_t)w) & 15) BRAID_REFUSE("gemm_heads_mma: operands must start on 16 bytes");
    if (((uintptr_t)out & 3) != 0) BRAID_REFUSE("gemm_heads_mma: the output must start on 4 bytes");
    cudaStream_t s = (cudaStream_t)stream;
    const int bm = n_rows <= 16 ? 16 : 64;
    dim3 grid((J + 63) / 64, (n_rows + bm - 1) / bm, heads);
    if (grid.y > 65535 || grid.z > 65535) BRAID_REFUSE("gemm_heads_mma: %d rows x %d heads exceed the grid limit", n_rows, heads);
    if (bm == 16)
        braid_launch(gemm_heads_mma_kernel<16>, grid, dim3(128), (size_t)MmaTile<16, 64, 1, 4, 1>::SMEM_BYTES, s,
                     (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate, n_rows, J, K,
                     ldx, hsx, ldo, hso, ldg, mult);
    else
        braid_launch(gemm_heads_mma_kernel<64>, grid, dim3(128), (size_t)MmaTile<64, 64, 2, 2, 1>::SMEM_BYTES, s,
                     (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate, n_rows, J, K,
                     ldx, hsx, ldo, hso, ldg, mult);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ plain attention over the latent cache
// One warp per (token, head).  s_j = (q~ . row_j) * scale over all D numbers of row j; online softmax;
// out = sum_j p_j row_j[0:rank] / sum_j p_j.  Key j is visible to the query at position p iff j <= p and,
// with a window w > 0, p - j < w.
struct AttnLatentArgs {
    const void* q;            // [rows, heads, D] at q + row*ldq + head*D
    void* out;                // [rows, heads, rank] at out + row*ldo + head*rank
    const void* cache;        // [pages][page_size][D]
    const int* page_table;
    const int* positions;
    const int* token_seq;
    long long ldq, ldo;
    int rows, heads, D, rank, page_size, table_cols, num_pages, window;
    float scale;
    int* error_flag;
};

#define ATTN_LATENT_WARPS 4

template <typename T, int NACC>
__global__ void __launch_bounds__(ATTN_LATENT_WARPS * 32)
attn_latent_simple_kernel(AttnLatentArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];                  // [warps][D] queries, [warps][32] probabilities
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* qs = smem + warp * a.D;
    float* ps = smem + ATTN_LATENT_WARPS * a.D + warp * 32;
    const long long item = (long long)blockIdx.x * ATTN_LATENT_WARPS + warp;
    if (item >= (long long)a.rows * a.heads) return;
    const int row = (int)(item / a.heads), head = (int)(item - (long long)row * a.heads);
    T* o = (T*)a.out + (size_t)row * a.ldo + (size_t)head * a.rank;
    const int seq = a.token_seq[row];
    if (seq < 0) {
        for (int d = lane; d < a.rank; d += 32) o[d] = from_f32<T>(0.f);
        return;
    }
    const int pos = a.positions[row];
    const T* q = (const T*)a.q + (size_t)row * a.ldq + (size_t)head * a.D;
    for (int d = lane; d < a.D; d += 32) qs[d] = to_f32(q[d]);
    __syncwarp();
    const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    float m = -INFINITY, l = 0.f;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    const int* table = a.page_table + (size_t)seq * a.table_cols;
    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        const T* krow = nullptr;
        if (j <= pos) {
            const int block = j / a.page_size, off = j - block * a.page_size;
            int page = (block < a.table_cols) ? table[block] : -1;
            if (page < 0 || page >= a.num_pages) {
                atomicExch(a.error_flag, 1);
                page = 0;
            }
            krow = (const T*)a.cache + ((size_t)page * a.page_size + off) * a.D;
            float dot = 0.f;
            for (int d = 0; d < a.D; ++d) dot = fmaf(qs[d], to_f32(krow[d]), dot);
            s = dot * a.scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float p = (j <= pos) ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
        m = m_new;
        ps[lane] = p;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= corr;
        const int n_valid = min(32, pos - j0 + 1);
        for (int jj = 0; jj < n_valid; ++jj) {
            const T* vr = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)krow, jj);
            const float pj = ps[jj];
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < a.rank) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
        __syncwarp();
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < a.rank) o[d] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T>
static cudaError_t launch_attn_latent_simple(const AttnLatentArgs& a, int blocks, size_t smem, cudaStream_t s) {
    const dim3 g(blocks), b(ATTN_LATENT_WARPS * 32);
    if (a.rank <= 64) return braid_launch(attn_latent_simple_kernel<T, 2>, g, b, smem, s, a);
    if (a.rank <= 128) return braid_launch(attn_latent_simple_kernel<T, 4>, g, b, smem, s, a);
    if (a.rank <= 256) return braid_launch(attn_latent_simple_kernel<T, 8>, g, b, smem, s, a);
    if (a.rank <= 512) return braid_launch(attn_latent_simple_kernel<T, 16>, g, b, smem, s, a);
    return braid_launch(attn_latent_simple_kernel<T, 32>, g, b, smem, s, a);
}

extern "C" int braid_attn_latent_simple(const void* q, void* out, int dtype, const void* cache, const int* page_table,
                                        const int* positions, const int* token_seq, long long ldq, long long ldo,
                                        int rows, int heads, int D, int rank, int page_size, int table_cols,
                                        int num_pages, int window, float scale, int* error_flag, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (!error_flag) BRAID_REFUSE("attn_latent_simple: error_flag is required");
    if (num_pages <= 0 || table_cols <= 0 || page_size <= 0) BRAID_REFUSE("attn_latent_simple: the cache has no pages");
    if (heads <= 0 || rank <= 0 || rank > D) BRAID_REFUSE("attn_latent_simple: heads=%d rank=%d D=%d", heads, rank, D);
    if (rank > 1024 || D > 2048) BRAID_REFUSE("attn_latent_simple: rank=%d (at most 1024), row size=%d (at most 2048)", rank, D);
    AttnLatentArgs a{q, out, cache, page_table, positions, token_seq, ldq, ldo, rows, heads, D, rank, page_size,
                     table_cols, num_pages, window, scale, error_flag};
    const long long items = (long long)rows * heads;
    const long long blocks = (items + ATTN_LATENT_WARPS - 1) / ATTN_LATENT_WARPS;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("attn_latent_simple: %lld (token, head) pairs exceed one launch", items);
    const size_t smem = (size_t)ATTN_LATENT_WARPS * (D + 32) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32) launch_attn_latent_simple<float>(a, (int)blocks, smem, s);
    else if (dtype == BRAID_BF16) launch_attn_latent_simple<__nv_bfloat16>(a, (int)blocks, smem, s);
    else BRAID_REFUSE("attn_latent_simple: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}
