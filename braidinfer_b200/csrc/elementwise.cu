// Row-wise kernels: embedding gather, RMSNorm, SiLU*up, residual add, rotary encoding
// with the write of keys and values into the paged cache.
//
// Formulas follow the reference ops they replace (by that project's paths):
//   embedding      kernels/megakernel_ops.hip:1757-1768 (a model's constant factor on the rows is applied here; 1 there)
//   rmsnorm        kernels/megakernel_ops.hip:862-904
//   silu * up      kernels/megakernel_ops.hip:374-407
//   residual add   kernels/megakernel_ops.hip:1185-1212
//   rotation       kernels/megakernel_ops.hip:2019-2030 (adjacent pairs)
//   cache write    kernels/op_kv_write_paged_batch.hip:38-78
// The residual stream is float32 in both run modes; sums of squares, rsqrt, angles,
// sin/cos and the residual sum are float32.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int n_tokens, int hidden, int vocab, float scale,
                             const T* __restrict__ pos_table, const int* __restrict__ positions, int max_pos, int* error_flag) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    int id = ids[t];
    const bool valid = (id >= 0 && id < vocab);
    const T* row = table + (size_t)(valid ? id : 0) * hidden;
    float* o = out + (size_t)t * hidden;
    if (pos_table) {
        // a learned vector a position, added unscaled in float32; a position past the table adds nothing and is flagged
        const int p = positions[t];
        const bool pv = p >= 0 && p < max_pos;
        if (!pv && valid && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
        const T* prow = pos_table + (size_t)(pv ? p : 0) * hidden;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x)
            o[i] = valid ? to_f32(row[i]) * scale + (pv ? to_f32(prow[i]) : 0.f) : 0.f;
        return;
    }
    // rows that start on 16 bytes and hold a whole number of 16-byte groups go group by group
    constexpr int VEC = 16 / sizeof(T);
    if (valid && hidden % VEC == 0 && (((uintptr_t)row | (uintptr_t)o) & 15) == 0) {
        for (int g = threadIdx.x; g < hidden / VEC; g += blockDim.x) {
            T v[VEC];
            *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(row + g * VEC);
#pragma unroll
            for (int e = 0; e < VEC; e += 4)
                *reinterpret_cast<float4*>(o + g * VEC + e) = make_float4(to_f32(v[e]) * scale, to_f32(v[e + 1]) * scale, to_f32(v[e + 2]) * scale, to_f32(v[e + 3]) * scale);
        }
        return;
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = valid ? to_f32(row[i]) * scale : 0.f;
}

extern "C" int braid_embed_pos(const void* table, int table_dtype, const int* ids, float* out, int n_tokens, int hidden,
                               int vocab, float scale, const void* pos_table, const int* positions, int max_pos,
                               int* error_flag, void* stream);
extern "C" int braid_embed(const void* table, int table_dtype, const int* ids, float* out,
                           int n_tokens, int hidden, int vocab, float scale, void* stream) {
    return braid_embed_pos(table, table_dtype, ids, out, n_tokens, hidden, vocab, scale, nullptr, nullptr, 0, nullptr, stream);
}

// The same with a second table [max_pos, hidden] of the table's element type: out[t] = table[ids[t]] * scale + pos_table[positions[t]].
extern "C" int braid_embed_pos(const void* table, int table_dtype, const int* ids, float* out, int n_tokens, int hidden,
                               int vocab, float scale, const void* pos_table, const int* positions, int max_pos,
                               int* error_flag, void* stream) {
    if (n_tokens <= 0) return BRAID_OK;
    if (pos_table && (!positions || max_pos <= 0)) BRAID_REFUSE("embed: a table of positions needs the rows' positions and its length");
    if (hidden <= 0 || vocab <= 0) BRAID_REFUSE("embed: hidden=%d vocab=%d must be positive", hidden, vocab);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == BRAID_F32)
        braid_launch(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)table, ids, out, n_tokens, hidden, vocab, scale, (const float*)pos_table, positions, max_pos, error_flag);
    else if (table_dtype == BRAID_BF16)
        braid_launch(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, (const __nv_bfloat16*)table, ids, out, n_tokens, hidden, vocab, scale, (const __nv_bfloat16*)pos_table, positions, max_pos, error_flag);
    else
        BRAID_REFUSE("embed: unknown table dtype code %d", table_dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ rmsnorm
// One block per output row.  `row_index` (may be null) picks the input row of each
// output row, which gathers the rows whose logits are wanted before the final norm.
// `w_offset` is added to every weight in float32 (1 for zero-centred weights).
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ row_index, int rows, int width, float eps, float w_offset) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int r = blockIdx.x;
    if (r >= rows) return;
    const int src = row_index ? row_index[r] : r;
    TO* o = out + (size_t)r * width;
    if (src < 0) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<TO>(0.f);
        return;
    }
    const float* xr = x + (size_t)src * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<TO>(xr[i] * scale * (to_f32(w[i]) + w_offset));
}

// Rows whose width is a multiple of 4 (and at most 4 * 8 * 512): one pass over x with
// 16-byte loads, the row kept in registers between the sum of squares and the scaling.
template <typename TW, typename TO, int PER>
__global__ void __launch_bounds__(512)
rmsnorm_vec_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                   const int* __restrict__ row_index, int rows, int width, float eps, float w_offset) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const int src = row_index ? row_index[r] : r;
    TO* o = out + (size_t)r * width;
    const int groups = width >> 2;
    if (src < 0) {
        for (int g = threadIdx.x; g < groups; g += blockDim.x)
            for (int e = 0; e < 4; ++e) o[g * 4 + e] = from_f32<TO>(0.f);
        return;
    }
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * width);
    float4 v[PER];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int g = threadIdx.x + i * blockDim.x;
        if (g < groups) {
            v[i] = xr[g];
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)width + eps);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int g = threadIdx.x + i * blockDim.x;
        if (g < groups) {
            const int c = g * 4;
            const float y0 = v[i].x * scale * (to_f32(w[c]) + w_offset), y1 = v[i].y * scale * (to_f32(w[c + 1]) + w_offset);
            const float y2 = v[i].z * scale * (to_f32(w[c + 2]) + w_offset), y3 = v[i].w * scale * (to_f32(w[c + 3]) + w_offset);
            if (sizeof(TO) == 2) {
                __nv_bfloat162 a = __floats2bfloat162_rn(y0, y1), b = __floats2bfloat162_rn(y2, y3);
                uint2 pk;
                pk.x = *reinterpret_cast<unsigned int*>(&a);
                pk.y = *reinterpret_cast<unsigned int*>(&b);
                *reinterpret_cast<uint2*>(o + c) = pk;
            } else {
                *reinterpret_cast<float4*>(o + c) = make_float4(y0, y1, y2, y3);
            }
        }
    }
}

extern "C" int braid_rmsnorm(const float* x, const void* w, int w_dtype, void* out, int out_dtype,
                             const int* row_index, int rows, int width, float eps, float w_offset, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (width <= 0) BRAID_REFUSE("rmsnorm: width=%d must be positive", width);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    const bool aligned = (width % 4 == 0) && (((uintptr_t)x & 15) == 0) && (((uintptr_t)out & 15) == 0);
    if (aligned && width <= 4 * 8 * threads) {
        const int per = (width / 4 + threads - 1) / threads;          // float4 groups a thread
#define BRAID_RMSV(TW, TO)                                                                                           \
        do {                                                                                                         \
            if (per <= 1) braid_launch(rmsnorm_vec_kernel<TW, TO, 1>, dim3(rows), dim3(threads), 0, s, x, (const TW*)w, (TO*)out, row_index, rows, width, eps, w_offset); \
            else if (per <= 2) braid_launch(rmsnorm_vec_kernel<TW, TO, 2>, dim3(rows), dim3(threads), 0, s, x, (const TW*)w, (TO*)out, row_index, rows, width, eps, w_offset); \
            else if (per <= 4) braid_launch(rmsnorm_vec_kernel<TW, TO, 4>, dim3(rows), dim3(threads), 0, s, x, (const TW*)w, (TO*)out, row_index, rows, width, eps, w_offset); \
            else braid_launch(rmsnorm_vec_kernel<TW, TO, 8>, dim3(rows), dim3(threads), 0, s, x, (const TW*)w, (TO*)out, row_index, rows, width, eps, w_offset); \
        } while (0)
        if (w_dtype == BRAID_F32 && out_dtype == BRAID_F32) BRAID_RMSV(float, float);
        else if (w_dtype == BRAID_F32 && out_dtype == BRAID_BF16) BRAID_RMSV(float, __nv_bfloat16);
        else if (w_dtype == BRAID_BF16 && out_dtype == BRAID_F32) BRAID_RMSV(__nv_bfloat16, float);
        else if (w_dtype == BRAID_BF16 && out_dtype == BRAID_BF16) BRAID_RMSV(__nv_bfloat16, __nv_bfloat16);
        else BRAID_REFUSE("rmsnorm: unknown dtype codes w=%d out=%d", w_dtype, out_dtype);
#undef BRAID_RMSV
        BRAID_LAUNCH_CHECK();
    }
#define BRAID_RMS(TW, TO) braid_launch(rmsnorm_kernel<TW, TO>, dim3(rows), dim3(threads), 0, s, x, (const TW*)w, (TO*)out, row_index, rows, width, eps, w_offset)
    if (w_dtype == BRAID_F32 && out_dtype == BRAID_F32) BRAID_RMS(float, float);
    else if (w_dtype == BRAID_F32 && out_dtype == BRAID_BF16) BRAID_RMS(float, __nv_bfloat16);
    else if (w_dtype == BRAID_BF16 && out_dtype == BRAID_F32) BRAID_RMS(__nv_bfloat16, float);
    else if (w_dtype == BRAID_BF16 && out_dtype == BRAID_BF16) BRAID_RMS(__nv_bfloat16, __nv_bfloat16);
    else BRAID_REFUSE("rmsnorm: unknown dtype codes w=%d out=%d", w_dtype, out_dtype);
#undef BRAID_RMS
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ act(gate) * up
// gu is [rows, 2*inter]: gate in columns [0, inter), up in [inter, 2*inter).  act: BRAID_ACT_*.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long total, int inter, int act) {
    pdl_trigger();
    pdl_wait();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / inter;
    const int c = (int)(i - r * inter);
    const float g = to_f32(gu[r * 2 * inter + c]);
    const float u = to_f32(gu[r * 2 * inter + inter + c]);
    out[i] = from_f32<T>(glu_act(g, act) * u);
}

extern "C" int braid_act_mul(const void* gu, void* out, int dtype, int rows, int inter, int act, void* stream);
extern "C" int braid_silu_mul(const void* gu, void* out, int dtype, int rows, int inter, void* stream) {
    return braid_act_mul(gu, out, dtype, rows, inter, BRAID_ACT_SILU, stream);
}

extern "C" int braid_act_mul(const void* gu, void* out, int dtype, int rows, int inter, int act, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (act < 0 || act >= BRAID_ACT_COUNT) BRAID_REFUSE("act_mul: unknown activation %d", act);
    if (inter <= 0) BRAID_REFUSE("silu_mul: inter=%d must be positive", inter);
    const long long total = (long long)rows * inter;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("silu_mul: %lld elements exceed one launch", total);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32) braid_launch(silu_mul_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, (const float*)gu, (float*)out, total, inter, act);
    else if (dtype == BRAID_BF16) braid_launch(silu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, total, inter, act);
    else BRAID_REFUSE("silu_mul: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ residual add
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ h, const T* __restrict__ delta, long long total) {
    pdl_trigger();
    pdl_wait();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) h[i] = h[i] + to_f32(delta[i]);
}

extern "C" int braid_residual_add(float* h, const void* delta, int delta_dtype, long long total, void* stream) {
    if (total <= 0) return BRAID_OK;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("residual_add: %lld elements exceed one launch", total);
    cudaStream_t s = (cudaStream_t)stream;
    if (delta_dtype == BRAID_F32) braid_launch(residual_add_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, h, (const float*)delta, total);
    else if (delta_dtype == BRAID_BF16) braid_launch(residual_add_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, h, (const __nv_bfloat16*)delta, total);
    else BRAID_REFUSE("residual_add: unknown dtype code %d", delta_dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ rotary + cache write
// qkv: [rows, (nqh + 2*nkh) * hd], heads in the order q..., k..., v....
// Queries are rotated in place.  Keys are rotated and written to the cache (and in
// place); values are copied to the cache.  A row whose token_seq is negative is
// padding and is left alone.  Cache of one layer: [page][2][nkh][page_size][hd].
struct RopeKvArgs {
    void* qkv;
    const float* inv_freq;       // [rope_dim / 2]
    const int* positions;        // [rows]
    const int* token_seq;        // [rows], index into the step's sequences, or -1
    const int* page_table;       // [n_seqs, table_cols], page of each logical block
    void* cache;                 // base of the layer's pool, or null (no write)
    int rows, nqh, nkh, hd, rope_dim, adjacent;
    int page_size, table_cols, num_pages;
    int* error_flag;
};

template <typename T>
__global__ void rope_kv_kernel(RopeKvArgs a) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int seq = a.token_seq[row];
    if (seq < 0) return;
    const int head = blockIdx.y;                     // [0, nqh + 2 nkh)
    const int pos = a.positions[row];
    const int width = (a.nqh + 2 * a.nkh) * a.hd;
    T* src = (T*)a.qkv + (size_t)row * width + (size_t)head * a.hd;
    const bool is_q = head < a.nqh;
    const bool is_k = !is_q && head < a.nqh + a.nkh;
    T* dst = nullptr;
    if (!is_q && a.cache) {
        const int kvh = is_k ? head - a.nqh : head - a.nqh - a.nkh;
        const int block = pos / a.page_size, off = pos - block * a.page_size;
        int page = (block < a.table_cols) ? a.page_table[(size_t)seq * a.table_cols + block] : -1;
        if (page < 0 || page >= a.num_pages) {
            if (threadIdx.x == 0) atomicExch(a.error_flag, 1);
            page = -1;
        }
        if (page >= 0)
            dst = (T*)a.cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * a.nkh + kvh) * a.page_size + off) * a.hd;
    }
    const int half = a.rope_dim / 2;
    if (is_q || is_k) {
        for (int p = threadIdx.x; p < half; p += blockDim.x) {
            const int i0 = a.adjacent ? 2 * p : p;
            const int i1 = a.adjacent ? 2 * p + 1 : p + half;
            const float ang = (float)pos * a.inv_freq[p];
            float sn, cs;
            sincosf(ang, &sn, &cs);
            const float x0 = to_f32(src[i0]), x1 = to_f32(src[i1]);
            const T y0 = from_f32<T>(x0 * cs - x1 * sn);
            const T y1 = from_f32<T>(x0 * sn + x1 * cs);
            src[i0] = y0;
            src[i1] = y1;
            if (dst) { dst[i0] = y0; dst[i1] = y1; }
        }
        if (dst)
            for (int i = a.rope_dim + threadIdx.x; i < a.hd; i += blockDim.x) dst[i] = src[i];
    } else if (dst) {
        for (int i = threadIdx.x; i < a.hd; i += blockDim.x) dst[i] = src[i];
    }
}

// One block per token; angles computed once per (token, pair) and shared by all heads;
// 16-byte loads and stores.  Needs head_dim and rope_dim to be multiples of 2 * VEC
// (VEC = 8 for bfloat16, 4 for float32) and 16-byte aligned rows.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_vec_kernel(RopeKvArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int VEC = 16 / sizeof(T);
    extern __shared__ float cs_sn[];                   // [rope_dim / 2] cosines, then sines
    const int row = blockIdx.x;
    const int seq = a.token_seq[row];
    if (seq < 0) return;
    const int pos = a.positions[row];
    const int half = a.rope_dim / 2;
    for (int p = threadIdx.x; p < half; p += blockDim.x) sincosf((float)pos * a.inv_freq[p], &cs_sn[half + p], &cs_sn[p]);
    const int width = (a.nqh + 2 * a.nkh) * a.hd;
    T* base = (T*)a.qkv + (size_t)row * width;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (a.cache) {
        const int block = pos / a.page_size, off = pos - block * a.page_size;
        int page = (block < a.table_cols) ? a.page_table[(size_t)seq * a.table_cols + block] : -1;
        if (page < 0 || page >= a.num_pages) {
            if (threadIdx.x == 0) atomicExch(a.error_flag, 1);
        } else {
            kdst = (T*)a.cache + (((size_t)page * 2) * a.nkh * a.page_size + off) * a.hd;       // + kvh * page_size * hd
            vdst = kdst + (size_t)a.nkh * a.page_size * a.hd;
        }
    }
    __syncthreads();
    const int rot_vecs = a.adjacent ? a.rope_dim / VEC : half / VEC;      // vectors a head's rotation takes
    const int pass_vecs = (a.hd - a.rope_dim) / VEC;                      // unrotated tail of a q/k head
    const int qk_heads = a.nqh + a.nkh;
    const int per_head = rot_vecs + pass_vecs;
    for (int item = threadIdx.x; item < qk_heads * per_head; item += blockDim.x) {
        const int head = item / per_head, j = item - head * per_head;
        T* h = base + (size_t)head * a.hd;
        T* dst = (head >= a.nqh && kdst) ? kdst + (size_t)(head - a.nqh) * a.page_size * a.hd : nullptr;
        if (j >= rot_vecs) {                            // tail beyond rope_dim: keys copy through to the cache
            const int i0 = a.rope_dim + (j - rot_vecs) * VEC;
            if (dst) *reinterpret_cast<uint4*>(dst + i0) = *reinterpret_cast<const uint4*>(h + i0);
            continue;
        }
        T x0[VEC], x1[VEC];
        if (a.adjacent) {
            const int i0 = j * VEC;                     // VEC / 2 pairs (2p, 2p + 1)
            *reinterpret_cast<uint4*>(x0) = *reinterpret_cast<const uint4*>(h + i0);
#pragma unroll
            for (int e = 0; e < VEC; e += 2) {
                const int p = (i0 + e) >> 1;
                const float c = cs_sn[p], sn = cs_sn[half + p];
                const float u = to_f32(x0[e]), v = to_f32(x0[e + 1]);
                x0[e] = from_f32<T>(u * c - v * sn);
                x0[e + 1] = from_f32<T>(u * sn + v * c);
            }
            *reinterpret_cast<uint4*>(h + i0) = *reinterpret_cast<const uint4*>(x0);
            if (dst) *reinterpret_cast<uint4*>(dst + i0) = *reinterpret_cast<const uint4*>(x0);
        } else {
            const int i0 = j * VEC;                     // VEC pairs (p, p + half)
            *reinterpret_cast<uint4*>(x0) = *reinterpret_cast<const uint4*>(h + i0);
            *reinterpret_cast<uint4*>(x1) = *reinterpret_cast<const uint4*>(h + i0 + half);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float c = cs_sn[i0 + e], sn = cs_sn[half + i0 + e];
                const float u = to_f32(x0[e]), v = to_f32(x1[e]);
                x0[e] = from_f32<T>(u * c - v * sn);
                x1[e] = from_f32<T>(u * sn + v * c);
            }
            *reinterpret_cast<uint4*>(h + i0) = *reinterpret_cast<const uint4*>(x0);
            *reinterpret_cast<uint4*>(h + i0 + half) = *reinterpret_cast<const uint4*>(x1);
            if (dst) {
                *reinterpret_cast<uint4*>(dst + i0) = *reinterpret_cast<const uint4*>(x0);
                *reinterpret_cast<uint4*>(dst + i0 + half) = *reinterpret_cast<const uint4*>(x1);
            }
        }
    }
    if (vdst) {
        const int hv = a.hd / VEC;
        const T* vsrc = base + (size_t)qk_heads * a.hd;
        for (int item = threadIdx.x; item < a.nkh * hv; item += blockDim.x) {
            const int kvh = item / hv, j = item - kvh * hv;
            *reinterpret_cast<uint4*>(vdst + (size_t)kvh * a.page_size * a.hd + j * VEC) =
                *reinterpret_cast<const uint4*>(vsrc + (size_t)kvh * a.hd + j * VEC);
        }
    }
}

extern "C" int braid_rope_kv_write(void* qkv, int dtype, const float* inv_freq, const int* positions,
                                   const int* token_seq, const int* page_table, void* cache,
                                   int rows, int nqh, int nkh, int hd, int rope_dim, int adjacent,
                                   int page_size, int table_cols, int num_pages, int* error_flag,
                                   void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (nqh <= 0 || nkh <= 0 || hd <= 0) BRAID_REFUSE("rope_kv_write: heads/head_dim must be positive");
    if (rope_dim < 0 || rope_dim > hd || (rope_dim & 1)) BRAID_REFUSE("rope_kv_write: rope_dim=%d must be even and <= head_dim=%d", rope_dim, hd);
    if (nqh + 2 * nkh > 65535) BRAID_REFUSE("rope_kv_write: %d heads exceed the grid limit", nqh + 2 * nkh);
    RopeKvArgs a{qkv, inv_freq, positions, token_seq, page_table, cache, rows, nqh, nkh, hd, rope_dim, adjacent,
                 page_size, table_cols, num_pages, error_flag};
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = dtype == BRAID_F32 ? 4 : 8;
    if ((dtype == BRAID_F32 || dtype == BRAID_BF16) && hd % (2 * vec) == 0 && rope_dim % (2 * vec) == 0 &&
        (((uintptr_t)qkv | (uintptr_t)cache) & 15) == 0) {
        const size_t smem = (size_t)rope_dim * sizeof(float);
        if (dtype == BRAID_F32) braid_launch(rope_kv_vec_kernel<float>, dim3(rows), dim3(128), smem, s, a);
        else braid_launch(rope_kv_vec_kernel<__nv_bfloat16>, dim3(rows), dim3(128), smem, s, a);
        BRAID_LAUNCH_CHECK();
    }
    dim3 grid(rows, nqh + 2 * nkh);
    const int threads = hd >= 128 ? 64 : 32;
    if (dtype == BRAID_F32) braid_launch(rope_kv_kernel<float>, dim3(grid), dim3(threads), 0, s, a);
    else if (dtype == BRAID_BF16) braid_launch(rope_kv_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, s, a);
    else BRAID_REFUSE("rope_kv_write: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ head norm + rotary + cache write
// For mixers that norm every query and key head before the rotation (RMS norm over the head with a
// weight of head_dim numbers shared by all heads) and, optionally, keep the key AS PROJECTED (before
// norm and rotation) as the value.  qk: [rows, row_stride], query heads then key heads (then value
// heads unless value_is_key).  One warp per (row, head): queries are normed and rotated in place;
// keys are normed, rotated, written in place and to the cache's key plane; the value plane takes the
// value head, or the key head as it came in.  The rotation turns the first rope_dim numbers of a head,
// pair (2p, 2p+1) if adjacent else (p, p + rope_dim/2), by angle pos * inv_freq[p]; sine and cosine
// are multiplied by `amp` (1 for a plain rotation).  Norm, angles and rotation are float32.
struct HeadNormRopeArgs {
    void* qk;
    long long row_stride;
    const void* q_w;             // [hd] or null (no norm on queries)
    const void* k_w;             // [hd] or null
    const float* inv_freq;       // [rope_dim / 2]
    const int* positions;
    const int* token_seq;
    const int* page_table;
    void* cache;                 // [page][2][nkh][page_size][hd] or null
    int rows, nqh, nkh, hd, rope_dim, adjacent, value_is_key;
    int page_size, table_cols, num_pages;
    float eps, amp;
    int* error_flag;
};

#define HEAD_NORM_MAX_HD 512
#define HEAD_NORM_WARPS 4
template <typename T> struct Pair2;
template <> struct Pair2<float> { using type = float2; };
template <> struct Pair2<__nv_bfloat16> { using type = __nv_bfloat162; };
__device__ __forceinline__ float2 pair_to_f32(float2 v) { return v; }
__device__ __forceinline__ float2 pair_to_f32(__nv_bfloat162 v) { return __bfloat1622float2(v); }
template <typename P> __device__ __forceinline__ P pair_from_f32(float a, float b);
template <> __device__ __forceinline__ float2 pair_from_f32<float2>(float a, float b) { return make_float2(a, b); }
template <> __device__ __forceinline__ __nv_bfloat162 pair_from_f32<__nv_bfloat162>(float a, float b) { return __floats2bfloat162_rn(a, b); }

// A warp a (row, head); the warps of a CTA take neighbouring heads of one row.  A lane holds whole neighbouring pairs
// (2p, 2p+1), p = lane, lane + 32, ...; PAIRS says whether they can be moved as one word (even head size and strides).
// (One CTA a row with sine and cosine shared by its heads was measured too: a warp then walks several heads one
// after the other, each a chain of load, sum, rotation and store, and the kernel took 1.5 times as long.)
template <typename T, bool PAIRS>
__global__ void __launch_bounds__(HEAD_NORM_WARPS * 32)
head_norm_rope_kv_kernel(HeadNormRopeArgs a) {
    pdl_trigger();
    pdl_wait();
    using P2 = typename Pair2<T>::type;
    __shared__ float stage[HEAD_NORM_WARPS][HEAD_NORM_MAX_HD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = a.nqh + (a.value_is_key ? a.nkh : 2 * a.nkh);
    const int per_row = (heads + HEAD_NORM_WARPS - 1) / HEAD_NORM_WARPS;          // CTAs a row
    const int row = blockIdx.x / per_row;
    const int head = (blockIdx.x - row * per_row) * HEAD_NORM_WARPS + warp;
    if (head >= heads) return;
    const int seq = a.token_seq[row];
    if (seq < 0) return;
    const int pos = a.positions[row];
    const int half = a.rope_dim / 2;
    T* kbase = nullptr;                                    // the row's place in the key plane, kv head 0
    if (a.cache) {
        const int block = pos / a.page_size, off = pos - block * a.page_size;
        const int page = (block < a.table_cols) ? a.page_table[(size_t)seq * a.table_cols + block] : -1;
        if (page < 0 || page >= a.num_pages) {
            if (lane == 0) atomicExch(a.error_flag, 1);
        } else {
            kbase = (T*)a.cache + (((size_t)page * 2) * a.nkh * a.page_size + off) * a.hd;
        }
    }
    const size_t plane = (size_t)a.nkh * a.page_size * a.hd, head_step = (size_t)a.page_size * a.hd;
    constexpr int NP = HEAD_NORM_MAX_HD / 64;             // pairs a lane
    {
        const bool is_q = head < a.nqh, is_k = !is_q && head < a.nqh + a.nkh;
        T* src = (T*)a.qk + (size_t)row * a.row_stride + (size_t)head * a.hd;
        T* kdst = nullptr;
        T* vdst = nullptr;
        if (!is_q && kbase) {
            const int kvh = is_k ? head - a.nqh : head - a.nqh - a.nkh;
            if (is_k) { kdst = kbase + kvh * head_step; if (a.value_is_key) vdst = kdst + plane; }
            else vdst = kbase + plane + kvh * head_step;
        }
        float x0[NP], x1[NP];
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < NP; ++e) {
            const int i = 2 * (lane + 32 * e);
            x0[e] = x1[e] = 0.f;
            if (PAIRS) {
                if (i < a.hd) {
                    const P2 raw = *reinterpret_cast<const P2*>(src + i);
                    if (vdst) *reinterpret_cast<P2*>(vdst + i) = raw;
                    const float2 f = pair_to_f32(raw);
                    x0[e] = f.x; x1[e] = f.y;
                }
            } else {
                if (i < a.hd) { const T r0 = src[i]; if (vdst) vdst[i] = r0; x0[e] = to_f32(r0); }
                if (i + 1 < a.hd) { const T r1 = src[i + 1]; if (vdst) vdst[i + 1] = r1; x1[e] = to_f32(r1); }
            }
            ss = fmaf(x0[e], x0[e], fmaf(x1[e], x1[e], ss));
        }
        if (!is_q && !is_k) return;
        const void* wv = is_q ? a.q_w : a.k_w;
        if (wv) {
            ss = warp_sum(ss);
            const float r = 1.f / sqrtf(ss / (float)a.hd + a.eps);
#pragma unroll
            for (int e = 0; e < NP; ++e) {
                const int i = 2 * (lane + 32 * e);
                if (i < a.hd) x0[e] = x0[e] * r * to_f32(((const T*)wv)[i]);
                if (i + 1 < a.hd) x1[e] = x1[e] * r * to_f32(((const T*)wv)[i + 1]);
            }
        }
        if (a.adjacent) {
#pragma unroll
            for (int e = 0; e < NP; ++e) {
                const int p = lane + 32 * e;
                if (p < half) {
                    float sn, cs;
                    sincosf((float)pos * a.inv_freq[p], &sn, &cs);
                    sn *= a.amp; cs *= a.amp;
                    const float u = x0[e], v = x1[e];
                    x0[e] = u * cs - v * sn;
                    x1[e] = v * cs + u * sn;
                }
            }
        } else if (half > 0) {
            // pairs (p, p + half) lie in different lanes: through shared memory
            float* st = stage[warp];
#pragma unroll
            for (int e = 0; e < NP; ++e) {
                const int i = 2 * (lane + 32 * e);
                if (i < a.hd) st[i] = x0[e];
                if (i + 1 < a.hd) st[i + 1] = x1[e];
            }
            __syncwarp();
#pragma unroll
            for (int e = 0; e < NP; ++e) {
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const int i = 2 * (lane + 32 * e) + b;
                    if (i < a.rope_dim) {
                        const int p = i < half ? i : i - half;
                        float sn, cs;
                        sincosf((float)pos * a.inv_freq[p], &sn, &cs);
                        sn *= a.amp; cs *= a.amp;
                        const float y = i < half ? st[i] * cs - st[i + half] * sn : st[i] * cs + st[i - half] * sn;
                        if (b) x1[e] = y; else x0[e] = y;
                    }
                }
            }
            __syncwarp();
        }
#pragma unroll
        for (int e = 0; e < NP; ++e) {
            const int i = 2 * (lane + 32 * e);
            if (PAIRS) {
                if (i < a.hd) {
                    const P2 y = pair_from_f32<P2>(x0[e], x1[e]);
                    *reinterpret_cast<P2*>(src + i) = y;
                    if (kdst) *reinterpret_cast<P2*>(kdst + i) = y;
                }
            } else {
                if (i < a.hd) { const T y = from_f32<T>(x0[e]); src[i] = y; if (kdst) kdst[i] = y; }
                if (i + 1 < a.hd) { const T y = from_f32<T>(x1[e]); src[i + 1] = y; if (kdst) kdst[i + 1] = y; }
            }
        }
    }
}

// The same for neighbouring pairs (or no rotation) with 16 bytes a lane: LPH lanes a head (LPH x 16 bytes hold the
// head), so a warp takes 32 / LPH heads of a row.  For head sizes and strides that allow aligned 16-byte moves.
template <typename T, int LPH>
__global__ void __launch_bounds__(128)
head_norm_rope_kv_vec_kernel(HeadNormRopeArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int VEC = 16 / sizeof(T), HPC = 128 / LPH;
    const int sub = threadIdx.x / LPH, l = threadIdx.x % LPH;
    const int heads = a.nqh + (a.value_is_key ? a.nkh : 2 * a.nkh);
    const int per_row = (heads + HPC - 1) / HPC;
    const int row = blockIdx.x / per_row;
    const int head = (blockIdx.x - row * per_row) * HPC + sub;
    const int seq = a.token_seq[row];
    if (seq < 0) return;                                   // the whole CTA: one row
    const int pos = a.positions[row];
    const int i0 = l * VEC;
    const bool in = head < heads && i0 < a.hd;             // lanes that hold nothing still take part in the shuffles
    const bool is_q = head < a.nqh, is_k = !is_q && head < a.nqh + a.nkh;
    T* src = (T*)a.qk + (size_t)row * a.row_stride + (size_t)head * a.hd + i0;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (in && !is_q && a.cache) {
        const int block = pos / a.page_size, off = pos - block * a.page_size;
        const int page = (block < a.table_cols) ? a.page_table[(size_t)seq * a.table_cols + block] : -1;
        if (page < 0 || page >= a.num_pages) {
            if (l == 0) atomicExch(a.error_flag, 1);
        } else {
            const int kvh = is_k ? head - a.nqh : head - a.nqh - a.nkh;
            T* kplane = (T*)a.cache + ((((size_t)page * 2) * a.nkh + kvh) * a.page_size + off) * a.hd + i0;
            T* vplane = kplane + (size_t)a.nkh * a.page_size * a.hd;
            if (is_k) { kdst = kplane; if (a.value_is_key) vdst = vplane; }
            else vdst = vplane;
        }
    }
    T raw[VEC];
    float x[VEC];
    if (in) *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(src);
    if (vdst) *reinterpret_cast<uint4*>(vdst) = *reinterpret_cast<const uint4*>(raw);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        x[e] = in ? to_f32(raw[e]) : 0.f;
        ss = fmaf(x[e], x[e], ss);
    }
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!in || (!is_q && !is_k)) return;
    const void* wv = is_q ? a.q_w : a.k_w;
    if (wv) {
        const float r = 1.f / sqrtf(ss / (float)a.hd + a.eps);
        T w[VEC];
        *reinterpret_cast<uint4*>(w) = *reinterpret_cast<const uint4*>((const T*)wv + i0);
#pragma unroll
        for (int e = 0; e < VEC; ++e) x[e] = x[e] * r * to_f32(w[e]);
    }
    const int half = a.rope_dim / 2;
#pragma unroll
    for (int e = 0; e < VEC; e += 2) {
        const int p = (i0 + e) >> 1;
        if (p < half) {
            float sn, cs;
            sincosf((float)pos * a.inv_freq[p], &sn, &cs);
            sn *= a.amp; cs *= a.amp;
            const float u = x[e], v = x[e + 1];
            x[e] = u * cs - v * sn;
            x[e + 1] = v * cs + u * sn;
        }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) raw[e] = from_f32<T>(x[e]);
    *reinterpret_cast<uint4*>(src) = *reinterpret_cast<const uint4*>(raw);
    if (kdst) *reinterpret_cast<uint4*>(kdst) = *reinterpret_cast<const uint4*>(raw);
}

template <typename T>
static bool launch_head_norm_vec(const HeadNormRopeArgs& a, int heads, cudaStream_t s) {
    constexpr int VEC = 16 / sizeof(T);
    const int lanes = (a.hd + VEC - 1) / VEC;
#define HN_LAUNCH(LPH)                                                                                        \
    do {                                                                                                      \
        const int hpc = 128 / LPH;                                                                            \
        const long long blocks = (long long)a.rows * ((heads + hpc - 1) / hpc);                               \
        if (blocks > 0x7fffffffLL) return false;                                                              \
        braid_launch(head_norm_rope_kv_vec_kernel<T, LPH>, dim3((unsigned)blocks), dim3(128), 0, s, a);       \
        return true;                                                                                          \
    } while (0)
    if (lanes <= 4) HN_LAUNCH(4);
    if (lanes <= 8) HN_LAUNCH(8);
    if (lanes <= 16) HN_LAUNCH(16);
    if (lanes <= 32) HN_LAUNCH(32);
#undef HN_LAUNCH
    return false;
}

extern "C" int braid_head_norm_rope_kv(void* qk, long long row_stride, int dtype, const void* q_w, const void* k_w,
                                       const float* inv_freq, const int* positions, const int* token_seq,
                                       const int* page_table, void* cache, int rows, int nqh, int nkh, int hd,
                                       int rope_dim, int adjacent, int value_is_key, int page_size, int table_cols,
                                       int num_pages, float eps, float amp, int* error_flag, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (nqh <= 0 || nkh <= 0 || hd <= 0 || hd > HEAD_NORM_MAX_HD)
        BRAID_REFUSE("head_norm_rope_kv: heads must be positive and head_dim=%d at most %d", hd, HEAD_NORM_MAX_HD);
    if (rope_dim < 0 || rope_dim > hd || (rope_dim & 1)) BRAID_REFUSE("head_norm_rope_kv: rope_dim=%d must be even and <= head_dim=%d", rope_dim, hd);
    HeadNormRopeArgs a{qk, row_stride, q_w, k_w, inv_freq, positions, token_seq, page_table, cache, rows, nqh, nkh, hd,
                       rope_dim, adjacent, value_is_key, page_size, table_cols, num_pages, eps, amp, error_flag};
    cudaStream_t s = (cudaStream_t)stream;
    const int esize = dtype == BRAID_F32 ? 4 : 2;
    // pairs move as one word where every head starts on a pair's boundary, in the rows and in the cache
    const bool pairs = (hd % 2 == 0) && (row_stride % 2 == 0) && (((uintptr_t)qk | (uintptr_t)cache) % (2 * esize) == 0);
    const int n_heads = nqh + (value_is_key ? nkh : 2 * nkh);
    const int vec = 16 / esize;
    // 16 bytes a lane where the heads, the rows, the norm weights and the cache allow aligned moves and pairs are neighbours
    const bool wide = (adjacent || rope_dim == 0) && hd % vec == 0 && row_stride % vec == 0 &&
                      (((uintptr_t)qk | (uintptr_t)cache | (uintptr_t)q_w | (uintptr_t)k_w) & 15) == 0;
    if (wide && (dtype == BRAID_F32 || dtype == BRAID_BF16)) {
        const bool done = dtype == BRAID_F32 ? launch_head_norm_vec<float>(a, n_heads, s) : launch_head_norm_vec<__nv_bfloat16>(a, n_heads, s);
        if (done) BRAID_LAUNCH_CHECK();
    }
    const long long blocks = (long long)rows * ((n_heads + HEAD_NORM_WARPS - 1) / HEAD_NORM_WARPS);
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("head_norm_rope_kv: %lld (row, head) pairs exceed one launch", (long long)rows * n_heads);
    const dim3 grid((unsigned)blocks), block(HEAD_NORM_WARPS * 32);
    if (dtype == BRAID_F32) {
        if (pairs) braid_launch(head_norm_rope_kv_kernel<float, true>, grid, block, 0, s, a);
        else braid_launch(head_norm_rope_kv_kernel<float, false>, grid, block, 0, s, a);
    } else if (dtype == BRAID_BF16) {
        if (pairs) braid_launch(head_norm_rope_kv_kernel<__nv_bfloat16, true>, grid, block, 0, s, a);
        else braid_launch(head_norm_rope_kv_kernel<__nv_bfloat16, false>, grid, block, 0, s, a);
    } else BRAID_REFUSE("head_norm_rope_kv: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ casts
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long total) {
    pdl_trigger();
    pdl_wait();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = from_f32<TO>(to_f32(in[i]));
}

extern "C" int braid_cast(const void* in, int in_dtype, void* out, int out_dtype, long long total, void* stream) {
    if (total <= 0) return BRAID_OK;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("cast: %lld elements exceed one launch", total);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == BRAID_F32 && out_dtype == BRAID_BF16) braid_launch(cast_kernel<float, __nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, (const float*)in, (__nv_bfloat16*)out, total);
    else if (in_dtype == BRAID_BF16 && out_dtype == BRAID_F32) braid_launch(cast_kernel<__nv_bfloat16, float>, dim3((int)blocks), dim3(threads), 0, s, (const __nv_bfloat16*)in, (float*)out, total);
    else BRAID_REFUSE("cast: unsupported dtype codes %d -> %d", in_dtype, out_dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ int32 gather
// dst[i] = src[index[i]]: feeds the tokens a sampler left on the device into the next step.
__global__ void gather_i32_kernel(const int* __restrict__ src, const int* __restrict__ index, int* __restrict__ dst, int n) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[index[i]];
}

extern "C" int braid_gather_i32(const int* src, const int* index, int* dst, int n, void* stream) {
    if (n <= 0) return BRAID_OK;
    braid_launch(gather_i32_kernel, dim3((n + 127) / 128), dim3(128), 0, (cudaStream_t)stream, src, index, dst, n);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ logit hash
// One 64-bit hash a row of float32 logits, for finding the first step at which two runs part: for every
// element in order, h ^= its 32 bits; h *= 0x100000001b3, from h = 0xcbf29ce484222325 (the hash that the
// reference writes under BRAIDINFER_LOGIT_TRACE, crates/braidinfer-runtime/src/generate.rs:383-396).
// The chain is sequential, so one thread a row walks it; the block stages the row through shared memory.
#define HASH_CHUNK 4096
__global__ void logit_hash_kernel(const float* __restrict__ logits, long long ld, int vocab, unsigned long long* __restrict__ out) {
    __shared__ float chunk[HASH_CHUNK];
    pdl_trigger();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * ld;
    unsigned long long h = 0xcbf29ce484222325ull;
    for (int c0 = 0; c0 < vocab; c0 += HASH_CHUNK) {
        const int n = min(HASH_CHUNK, vocab - c0);
        for (int i = threadIdx.x; i < n; i += blockDim.x) chunk[i] = row[c0 + i];
        __syncthreads();
        if (threadIdx.x == 0)
            for (int i = 0; i < n; ++i) {
                h ^= (unsigned long long)__float_as_uint(chunk[i]);
                h *= 0x100000001b3ull;
            }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = h;
}

extern "C" int braid_logit_hash(const float* logits, long long ld, int rows, int vocab, unsigned long long* out, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (vocab <= 0 || ld < vocab) BRAID_REFUSE("logit_hash: vocab=%d, row stride=%lld", vocab, ld);
    braid_launch(logit_hash_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, logits, ld, vocab, out);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ heads without rotation: norm, temperature, cache write
// Rows of stacked heads [rows, row_stride]: nqh query heads of dk numbers, then nkh key heads of dk, then nkh value
// heads of dv.  With `unit`, every query and key head is divided by its root mean square, sqrt(mean(x^2) + eps)
// (no weight).  A query is then multiplied by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1), p the row's
// position (temp_every = 0: no such factor).  Queries go to q_out [rows, nqh * hd] and keys and values into the
// cache's planes [page][2][nkh][page_size][hd], all padded with zeros from their own size up to hd (a head size that
// the attention kernels take); zeros change neither a score nor a result's first dv numbers.  Padding rows get zero
// queries and write no cache.  One warp a (row, head); float32 arithmetic.
struct HeadPrepArgs {
    const void* src; long long row_stride;
    void* q_out;
    const int* positions; const int* token_seq; const int* page_table;
    void* cache;
    int rows, nqh, nkh, dk, dv, hd, unit;
    int page_size, table_cols, num_pages;
    float eps, temp_coef; int temp_every;
    int* error_flag;
    int vec8;              // 16 bytes a lane (bfloat16, aligned heads of up to 256 numbers)
};

template <typename T>
__global__ void __launch_bounds__(128)
head_prep_kv_kernel(HeadPrepArgs a) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = a.nqh + 2 * a.nkh;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)a.rows * heads) return;
    const int row = (int)(item / heads), head = (int)(item - (long long)row * heads);
    const int seq = a.token_seq[row];
    const bool is_q = head < a.nqh, is_k = !is_q && head < a.nqh + a.nkh;
    if (seq < 0) {
        if (is_q) {
            T* o = (T*)a.q_out + ((size_t)row * a.nqh + head) * a.hd;
            for (int c = lane; c < a.hd; c += 32) o[c] = from_f32<T>(0.f);
        }
        return;
    }
    const int d = is_q || is_k ? a.dk : a.dv;
    const size_t col0 = is_q ? (size_t)head * a.dk
                      : is_k ? (size_t)a.nqh * a.dk + (size_t)(head - a.nqh) * a.dk
                             : (size_t)(a.nqh + a.nkh) * a.dk + (size_t)(head - a.nqh - a.nkh) * a.dv;
    const T* src = (const T*)a.src + (size_t)row * a.row_stride + col0;
    const int pos = a.positions[row];
    float f = 1.f;
    if constexpr (sizeof(T) == 2) {
        // 16 bytes a lane, the head read once and kept: heads of up to 256 numbers whose rows and sizes keep every
        // head on a 16-byte boundary (the padded head then does too)
        if (a.vec8) {
            const int c = lane * 8;
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            if (c < d) raw = *reinterpret_cast<const uint4*>(src + c);
            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            float v[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 u = __bfloat1622float2(p2[j]); v[2 * j] = u.x; v[2 * j + 1] = u.y; }
            if ((is_q || is_k) && a.unit) {
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) ss = fmaf(v[j], v[j], ss);
                ss = warp_sum(ss);
                f = 1.f / sqrtf(ss / (float)d + a.eps);
            }
            if (is_q && a.temp_every > 0) f *= 1.f + a.temp_coef * logf((float)((pos + 1) / a.temp_every) + 1.f);
            T* dst8 = nullptr;
            if (is_q) {
                dst8 = (T*)a.q_out + ((size_t)row * a.nqh + head) * a.hd;
            } else if (a.cache) {
                const int kvh = is_k ? head - a.nqh : head - a.nqh - a.nkh;
                const int block = pos / a.page_size, off = pos - block * a.page_size;
                const int page = (block < a.table_cols) ? a.page_table[(size_t)seq * a.table_cols + block] : -1;
                if (page < 0 || page >= a.num_pages) {
                    if (lane == 0) atomicExch(a.error_flag, 1);
                    return;
                }
                dst8 = (T*)a.cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * a.nkh + kvh) * a.page_size + off) * a.hd;
            }
            if (!dst8 || c >= a.hd) return;
            uint4 packed;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
            for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[2 * j] * f, v[2 * j + 1] * f);
            *reinterpret_cast<uint4*>(dst8 + c) = packed;
            return;
        }
    }
    if ((is_q || is_k) && a.unit) {
        float ss = 0.f;
        for (int c = lane; c < d; c += 32) { const float v = to_f32(src[c]); ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        f = 1.f / sqrtf(ss / (float)d + a.eps);
    }
    if (is_q && a.temp_every > 0) f *= 1.f + a.temp_coef * logf((float)((pos + 1) / a.temp_every) + 1.f);
    T* dst = nullptr;
    if (is_q) {
        dst = (T*)a.q_out + ((size_t)row * a.nqh + head) * a.hd;
    } else if (a.cache) {
        const int kvh = is_k ? head - a.nqh : head - a.nqh - a.nkh;
        const int block = pos / a.page_size, off = pos - block * a.page_size;
        int page = (block < a.table_cols) ? a.page_table[(size_t)seq * a.table_cols + block] : -1;
        if (page < 0 || page >= a.num_pages) {
            if (lane == 0) atomicExch(a.error_flag, 1);
            return;
        }
        dst = (T*)a.cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * a.nkh + kvh) * a.page_size + off) * a.hd;
    }
    if (!dst) return;
    for (int c = lane; c < a.hd; c += 32) dst[c] = from_f32<T>(c < d ? to_f32(src[c]) * f : 0.f);
}

extern "C" int braid_head_prep_kv(const void* src, long long row_stride, int dtype, void* q_out, const int* positions,
                                  const int* token_seq, const int* page_table, void* cache, int rows, int nqh, int nkh,
                                  int dk, int dv, int hd, int unit, int page_size, int table_cols, int num_pages, float eps,
                                  float temp_coef, int temp_every, int* error_flag, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (nqh <= 0 || nkh <= 0 || dk <= 0 || dv <= 0 || hd < dk || hd < dv)
        BRAID_REFUSE("head_prep_kv: heads %d/%d of sizes %d and %d do not fit a padded head of %d", nqh, nkh, dk, dv, hd);
    if (cache && !page_table) BRAID_REFUSE("head_prep_kv: a cache write needs the step's page table");
    const int vec8 = dtype == BRAID_BF16 && hd <= 256 && !(dk & 7) && !(dv & 7) && !(hd & 7) && !(row_stride & 7) &&
                     !((uintptr_t)src & 15) && !((uintptr_t)q_out & 15) && !((uintptr_t)cache & 15);
    HeadPrepArgs a{src, row_stride, q_out, positions, token_seq, page_table, cache, rows, nqh, nkh, dk, dv, hd, unit,
                   page_size, table_cols, num_pages, eps, temp_coef, temp_every, error_flag, vec8};
    const long long blocks = ((long long)rows * (nqh + 2 * nkh) + 3) / 4;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("head_prep_kv: %d rows exceed one launch", rows);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32) braid_launch(head_prep_kv_kernel<float>, dim3((int)blocks), dim3(128), 0, s, a);
    else if (dtype == BRAID_BF16) braid_launch(head_prep_kv_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(128), 0, s, a);
    else BRAID_REFUSE("head_prep_kv: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ a gate a head on attention's result
// out[r, h * dv + c] = x[r, h * hd + c] * sigmoid(gate[r, h]) for c < dv: the first dv numbers of every padded head,
// times the head's gate (gate: a column block of the stacked projection, row stride gate_stride; null: no gate).
template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ gate, long long gate_stride,
                                 T* __restrict__ out, long long total, int heads, int hd, int dv) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int per_row = heads * dv;
    const long long r = i / per_row;
    const int rem = (int)(i - r * per_row), h = rem / dv, c = rem - h * dv;
    float v = to_f32(x[r * x_stride + (size_t)h * hd + c]);
    if (gate) v *= 1.f / (1.f + expf(-to_f32(gate[r * gate_stride + h])));
    out[i] = from_f32<T>(v);
}

extern "C" int braid_head_gate(const void* x, long long x_stride, const void* gate, long long gate_stride, void* out,
                               int dtype, int rows, int heads, int hd, int dv, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (heads <= 0 || dv <= 0 || hd < dv) BRAID_REFUSE("head_gate: %d heads of %d numbers in heads of %d", heads, dv, hd);
    const long long total = (long long)rows * heads * dv, blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("head_gate: %lld elements exceed one launch", total);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32)
        braid_launch(head_gate_kernel<float>, dim3((int)blocks), dim3(256), 0, s, (const float*)x, x_stride, (const float*)gate,
                     gate_stride, (float*)out, total, heads, hd, dv);
    else if (dtype == BRAID_BF16)
        braid_launch(head_gate_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, s, (const __nv_bfloat16*)x, x_stride,
                     (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, total, heads, hd, dv);
    else BRAID_REFUSE("head_gate: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ the clamped gated unit
// gu is [rows, 2 * inter]: gate in columns [0, inter), up in [inter, 2 * inter).
// g = min(gate, limit), u = clamp(up, -limit, limit); out = g * sigmoid(alpha * g) * (u + 1).
template <typename T>
__global__ void glu_clamp_kernel(const T* __restrict__ gu, T* __restrict__ out, long long total, int inter, float limit, float alpha) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / inter;
    const int c = (int)(i - r * inter);
    out[i] = from_f32<T>(glu_clamp_f32(to_f32(gu[r * 2 * inter + c]), to_f32(gu[r * 2 * inter + inter + c]), limit, alpha));
}

extern "C" int braid_glu_clamp(const void* gu, void* out, int dtype, int rows, int inter, float limit, float alpha, void* stream) {
    if (rows <= 0 || inter <= 0) return BRAID_OK;
    const long long total = (long long)rows * inter, blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("glu_clamp: %lld elements exceed one launch", total);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32) braid_launch(glu_clamp_kernel<float>, dim3((int)blocks), dim3(256), 0, s, (const float*)gu, (float*)out, total, inter, limit, alpha);
    else if (dtype == BRAID_BF16) braid_launch(glu_clamp_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, total, inter, limit, alpha);
    else BRAID_REFUSE("glu_clamp: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}
