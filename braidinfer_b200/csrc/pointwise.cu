// Element-wise kernels that models beside the dense Mistral decoder need: the Dynamic Tanh norm,
// the soft cap of logits, and the side-by-side copy of two residual streams into one product's input.
// All arithmetic is float32; inputs are the float32 residual stream or float32 logits.
#include "common.cuh"

// ------------------------------------------------------------------ Dynamic Tanh
// y[r, i] = tanh(alpha * (x[src(r), i] * in_scale)) * w[i] + b[i].  No mean and no variance: rows are
// independent element by element.  alpha is one stored scalar.  `row_index` (may be null) picks the input
// row of each output row; a negative index gives a row of zeros.  out may be x itself (TO = float).
template <typename TW, typename TO>
__global__ void dyt_kernel(const float* x, const TW* __restrict__ w, const TW* __restrict__ b,
                           const TW* __restrict__ alpha, TO* out, const int* __restrict__ row_index,
                           int rows, int width, float in_scale) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    if (r >= rows) return;
    const int src = row_index ? row_index[r] : r;
    TO* o = out + (size_t)r * width;
    if (src < 0) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<TO>(0.f);
        return;
    }
    const float a = to_f32(alpha[0]) ;
    const float* xr = x + (size_t)src * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        o[i] = from_f32<TO>(fmaf(tanhf(a * (xr[i] * in_scale)), to_f32(w[i]), to_f32(b[i])));
}

extern "C" int braid_dyt(const float* x, const void* w, const void* b, const void* alpha, int w_dtype,
                         void* out, int out_dtype, const int* row_index, int rows, int width, float in_scale,
                         void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (width <= 0) BRAID_REFUSE("dyt: width=%d must be positive", width);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : 128;
#define BRAID_DYT(TW, TO) braid_launch(dyt_kernel<TW, TO>, dim3(rows), dim3(threads), 0, s, x, (const TW*)w, (const TW*)b, (const TW*)alpha, (TO*)out, row_index, rows, width, in_scale)
    if (w_dtype == BRAID_F32 && out_dtype == BRAID_F32) BRAID_DYT(float, float);
    else if (w_dtype == BRAID_F32 && out_dtype == BRAID_BF16) BRAID_DYT(float, __nv_bfloat16);
    else if (w_dtype == BRAID_BF16 && out_dtype == BRAID_F32) BRAID_DYT(__nv_bfloat16, float);
    else if (w_dtype == BRAID_BF16 && out_dtype == BRAID_BF16) BRAID_DYT(__nv_bfloat16, __nv_bfloat16);
    else BRAID_REFUSE("dyt: unknown dtype codes w=%d out=%d", w_dtype, out_dtype);
#undef BRAID_DYT
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ soft cap
// x <- cap * tanh(x / cap), in place, float32.
__global__ void softcap_kernel(float* x, long long total, float cap, float inv_cap) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] = cap * tanhf(x[i] * inv_cap);
}

extern "C" int braid_softcap(float* x, long long total, float cap, void* stream) {
    if (total <= 0) return BRAID_OK;
    if (!(cap > 0.f)) BRAID_REFUSE("softcap: the cap must be positive, got %g", (double)cap);
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("softcap: %lld elements exceed one launch", total);
    braid_launch(softcap_kernel, dim3((int)blocks), dim3(threads), 0, (cudaStream_t)stream, x, total, cap, 1.f / cap);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ two streams side by side
// out[r, 0:w] = a[r, :], out[r, w:2w] = b[r, :], float32 in, TO out.
template <typename TO>
__global__ void concat2_kernel(const float* __restrict__ a, const float* __restrict__ b, TO* __restrict__ out,
                               long long total, int width) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / (2 * width);
    const int c = (int)(i - r * 2 * width);
    out[i] = from_f32<TO>(c < width ? a[r * width + c] : b[r * width + c - width]);
}

extern "C" int braid_concat2(const float* a, const float* b, void* out, int out_dtype, int rows, int width,
                             void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (width <= 0) BRAID_REFUSE("concat2: width=%d must be positive", width);
    const long long total = (long long)rows * 2 * width;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("concat2: %lld elements exceed one launch", total);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == BRAID_F32) braid_launch(concat2_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, a, b, (float*)out, total, width);
    else if (out_dtype == BRAID_BF16) braid_launch(concat2_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, a, b, (__nv_bfloat16*)out, total, width);
    else BRAID_REFUSE("concat2: unknown dtype code %d", out_dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ a layer's own token input
// g[r, j] = act(gate[r, j]) * table[token[r], col0 + j]: a gate computed from the stream, times the columns
// [col0, col0 + dim) of a token table's row.  float32 arithmetic; gate, table and g in the run's type.
template <typename T>
__global__ void act_mul_gather_kernel(const T* __restrict__ gate, long long gate_stride, const T* __restrict__ table,
                                      long long table_stride, const int* __restrict__ ids, int vocab, int col0,
                                      T* __restrict__ out, long long total, int dim, int act) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / dim;
    const int j = (int)(i - r * dim);
    int id = ids[r];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const float g = to_f32(gate[r * gate_stride + j]);
    out[i] = from_f32<T>(glu_act(g, act) * to_f32(table[(size_t)id * table_stride + col0 + j]));
}

extern "C" int braid_act_mul_gather(const void* gate, long long gate_stride, const void* table, long long table_stride,
                                    const int* ids, int vocab, int col0, void* out, int dtype, int rows, int dim, int act,
                                    void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (dim <= 0 || vocab <= 0 || col0 < 0) BRAID_REFUSE("act_mul_gather: dim=%d, vocab=%d, col0=%d", dim, vocab, col0);
    if (act < 0 || act >= BRAID_ACT_COUNT) BRAID_REFUSE("act_mul_gather: unknown activation %d", act);
    const long long total = (long long)rows * dim;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("act_mul_gather: %lld elements exceed one launch", total);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32)
        braid_launch(act_mul_gather_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, (const float*)gate, gate_stride,
                     (const float*)table, table_stride, ids, vocab, col0, (float*)out, total, dim, act);
    else if (dtype == BRAID_BF16)
        braid_launch(act_mul_gather_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, (const __nv_bfloat16*)gate,
                     gate_stride, (const __nv_bfloat16*)table, table_stride, ids, vocab, col0, (__nv_bfloat16*)out, total, dim, act);
    else BRAID_REFUSE("act_mul_gather: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

// h[r] += y[r] / sqrt(mean(y[r]^2) + eps) * (w + w_offset): an RMS norm of a branch's result (w_offset 0 for plain weights,
// 1 for zero-centred weights), added to the float32 stream.  y float32 [rows, width]; one CTA a row; sums in float32, the same order every time.
template <typename TW>
__global__ void __launch_bounds__(256)
rmsnorm_add_kernel(float* __restrict__ h, const float* __restrict__ y, const TW* __restrict__ w, int width, float eps, float w_offset) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { const float v = y[base + c]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) h[base + c] += y[base + c] * r * (to_f32(w[c]) + w_offset);
}

extern "C" int braid_rmsnorm_add(float* h, const float* y, const void* w, int w_dtype, int rows, int width, float eps,
                                 float w_offset, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (width <= 0) BRAID_REFUSE("rmsnorm_add: width=%d must be positive", width);
    cudaStream_t s = (cudaStream_t)stream;
    if (w_dtype == BRAID_F32) braid_launch(rmsnorm_add_kernel<float>, dim3(rows), dim3(256), 0, s, h, y, (const float*)w, width, eps, w_offset);
    else if (w_dtype == BRAID_BF16) braid_launch(rmsnorm_add_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, s, h, y, (const __nv_bfloat16*)w, width, eps, w_offset);
    else BRAID_REFUSE("rmsnorm_add: unknown dtype code %d", w_dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ a mix of the heads after the softmax
// Attention whose probabilities are mixed across the heads before they meet the values,
//     p'_h(i, j) = sum_g talk[h, g] p_g(i, j),      out_h(i) = sum_j p'_h(i, j) v_kv(h)(j),
// is linear in the probabilities, so out_h = sum_g talk[h, g] O[g, kv(h)] with O[g, c] = sum_j p_g(i, j) v_c(j): what the
// attention kernels leave at virtual head g * kv_heads + c when every query head reads the values of every kv head.
// src [rows, heads * kv_heads, hd] -> out [rows, heads, vd] (the first vd numbers of a head: heads may be padded).
// The sum over g is float32, in the order of g.
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
head_mix_kernel(const T* __restrict__ src, long long lds, const TW* __restrict__ talk, T* __restrict__ out,
                long long ldo, const int* __restrict__ token_seq, int heads, int kvh, int hd, int vd) {
    // one CTA a row and kv head c: the results of every head over c's values wait in shared memory, and the heads of
    // c's group each take their mix of them
    extern __shared__ float mix_slab[];                    // [heads][vd]
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, c = blockIdx.y;
    const bool padding = token_seq && token_seq[row] < 0;
    const int group = heads / kvh;
    const T* s = src + (size_t)row * lds;
    T* o = out + (size_t)row * ldo;
    // 16 bytes a thread where rows and heads allow it (bfloat16: eight numbers)
    constexpr int VEC = 16 / sizeof(T);
    const bool wide = sizeof(T) == 2 && hd % VEC == 0 && vd % VEC == 0 && lds % VEC == 0 && ldo % VEC == 0 &&
                      (((uintptr_t)src | (uintptr_t)out) & 15) == 0;
    if (!padding) {
        if (wide) {
            const int per = vd / VEC;
            for (int i = threadIdx.x; i < heads * per; i += blockDim.x) {
                const int g = i / per, d = (i - g * per) * VEC;
                T raw[VEC];
                *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(s + ((size_t)g * kvh + c) * hd + d);
#pragma unroll
                for (int e = 0; e < VEC; ++e) mix_slab[g * vd + d + e] = to_f32(raw[e]);
            }
        } else {
            for (int i = threadIdx.x; i < heads * vd; i += blockDim.x) {
                const int g = i / vd, d = i - g * vd;
                mix_slab[i] = to_f32(s[((size_t)g * kvh + c) * hd + d]);
            }
        }
    }
    __syncthreads();
    if (wide) {
        const int per = vd / VEC;
        for (int i = threadIdx.x; i < group * per; i += blockDim.x) {
            const int h = c * group + i / per, d = (i % per) * VEC;
            float acc[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
            if (!padding)
                for (int g = 0; g < heads; ++g) {
                    const float w = to_f32(talk[h * heads + g]);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) acc[e] = fmaf(w, mix_slab[g * vd + d + e], acc[e]);
                }
            T raw[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) raw[e] = from_f32<T>(acc[e]);
            *reinterpret_cast<uint4*>(o + (size_t)h * vd + d) = *reinterpret_cast<const uint4*>(raw);
        }
        return;
    }
    for (int i = threadIdx.x; i < group * vd; i += blockDim.x) {
        const int h = c * group + i / vd, d = i % vd;
        float acc = 0.f;
        if (!padding)
            for (int g = 0; g < heads; ++g) acc = fmaf(to_f32(talk[h * heads + g]), mix_slab[g * vd + d], acc);
        o[(size_t)h * vd + d] = from_f32<T>(acc);
    }
}

extern "C" int braid_head_mix(const void* src, long long lds, const void* talk, int talk_dtype, void* out, long long ldo,
                              int dtype, const int* token_seq, int rows, int heads, int kvh, int hd, int vd, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (heads <= 0 || kvh <= 0 || heads % kvh || vd <= 0 || vd > hd) BRAID_REFUSE("head_mix: heads=%d kv heads=%d head size=%d value size=%d", heads, kvh, hd, vd);
    const size_t smem = (size_t)heads * vd * sizeof(float);
    if (smem > 200 * 1024) BRAID_REFUSE("head_mix: %d heads of %d values are more than one block's shared memory holds", heads, vd);
    if (kvh > 65535) BRAID_REFUSE("head_mix: %d kv heads exceed the grid limit", kvh);
    cudaStream_t s = (cudaStream_t)stream;
#define BRAID_MIX(T, TW)                                                                                               \
    do {                                                                                                               \
        if (smem > 48 * 1024) {                                                                                        \
            cudaError_t e_ = cudaFuncSetAttribute(head_mix_kernel<T, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e_ != cudaSuccess) BRAID_REFUSE("head_mix: shared memory: %s", cudaGetErrorString(e_));                 \
        }                                                                                                              \
        braid_launch(head_mix_kernel<T, TW>, dim3(rows, kvh), dim3(128), smem, s, (const T*)src, lds, (const TW*)talk, \
                     (T*)out, ldo, token_seq, heads, kvh, hd, vd);                                                     \
    } while (0)
    if (dtype == BRAID_F32 && talk_dtype == BRAID_F32) BRAID_MIX(float, float);
    else if (dtype == BRAID_BF16 && talk_dtype == BRAID_BF16) BRAID_MIX(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == BRAID_BF16 && talk_dtype == BRAID_F32) BRAID_MIX(__nv_bfloat16, float);
    else BRAID_REFUSE("head_mix: unknown dtype codes rows=%d talk=%d", dtype, talk_dtype);
#undef BRAID_MIX
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ bias + xIELU
// out[r, j] = f(z[r, j] + b[j]) for j < J, with the two-piece activation
//     f(t) = softplus(p) t^2 + t / 2                           t > 0
//     f(t) = (1/2 + softplus(q)) (exp(t) - 1 - t) + t / 2      t <= 0
// whose two numbers (p, q) are stored with the layer (`pq`).  Columns J .. ldo of out are written as 1, 0, 0, ...: the
// product that reads out then adds its own bias as the weight column that meets the 1.  float32 arithmetic.
#define XIELU_SPAN 1024
template <typename T, typename TW>
__global__ void bias_xielu_kernel(const T* __restrict__ z, long long ldz, const TW* __restrict__ b, const TW* __restrict__ pq,
                                  T* __restrict__ out, long long ldo, int J, int cols) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;                            // blockIdx.y: a span of XIELU_SPAN columns
    const float p = to_f32(pq[0]), q = to_f32(pq[1]);
    const float ap = fmaxf(p, 0.f) + log1pf(expf(-fabsf(p)));
    const float aq = 0.5f + fmaxf(q, 0.f) + log1pf(expf(-fabsf(q)));
    const T* zr = z + (size_t)row * ldz;
    T* o = out + (size_t)row * ldo;
    const int j_end = min(cols, (int)(blockIdx.y + 1) * XIELU_SPAN);
    for (int j = blockIdx.y * XIELU_SPAN + threadIdx.x; j < j_end; j += blockDim.x) {
        float y;
        if (j < J) {
            const float t = to_f32(zr[j]) + to_f32(b[j]);
            y = t > 0.f ? fmaf(ap * t, t, 0.5f * t) : fmaf(aq, expm1f(t) - t, 0.5f * t);
        } else {
            y = j == J ? 1.f : 0.f;
        }
        o[j] = from_f32<T>(y);
    }
}

extern "C" int braid_bias_xielu(const void* z, long long ldz, const void* b, const void* pq, int w_dtype, void* out,
                                long long ldo, int dtype, int rows, int J, int cols, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (J <= 0 || cols < J || cols > ldo) BRAID_REFUSE("bias_xielu: %d numbers a row, %d columns written, rows of %lld", J, cols, ldo);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
#define BRAID_XI(T, TW) braid_launch(bias_xielu_kernel<T, TW>, dim3(rows, (cols + XIELU_SPAN - 1) / XIELU_SPAN), dim3(threads), 0, s, (const T*)z, ldz, (const TW*)b, (const TW*)pq, (T*)out, ldo, J, cols)
    if (dtype == BRAID_F32 && w_dtype == BRAID_F32) BRAID_XI(float, float);
    else if (dtype == BRAID_BF16 && w_dtype == BRAID_BF16) BRAID_XI(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == BRAID_BF16 && w_dtype == BRAID_F32) BRAID_XI(__nv_bfloat16, float);
    else BRAID_REFUSE("bias_xielu: unknown dtype codes rows=%d weights=%d", dtype, w_dtype);
#undef BRAID_XI
    BRAID_LAUNCH_CHECK();
}
