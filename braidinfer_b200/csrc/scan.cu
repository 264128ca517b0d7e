// Kernels of mixers that carry a fixed-size state from token to token instead of keys and values:
// a short causal convolution per channel, the linear recurrence S_t = diag(a_t) S_(t-1) + k_t v_t^T
// with o_t = S_t^T q_t (gated linear attention: a decay per key channel; state-space duality: one
// decay per head, a step size on the key and a skip term), and the gated RMS norms that follow them.
//
// A step's rows are packed sequence after sequence (q_start, q_len per sequence; a row's token_seq
// is its sequence or -1 for padding).  The state of a sequence lies in its slot of the cache's state
// area: `state` + slot * state_stride bytes; every kernel below is given the byte offset of its own
// part of it.  The state, the decays, step sizes, gates and norms are float32 whatever the run's
// element type; projections and the convolution's output are in the run's type T.
//
// A recurrence is walked token by token in the order of the sequence, so the state after a prompt
// does not depend on how the prompt was cut into steps: a step continues from the stored state with
// the very operations a longer step would have done.
#include "common.cuh"

// ------------------------------------------------------------------ causal convolution
// y[t, c] = act(b[c] + sum_j w[c, j] x[t - (taps - 1 - j), c]): the last column of w is the current
// token's.  Inputs before the step come from the state, which keeps a sequence's last taps - 1
// inputs (zeros before its start): state[i, c], i = taps - 2 the newest.
struct ConvArgs {
    const void* x;               // [rows, x_stride], channel c at column c
    long long x_stride;
    void* y;                     // [rows, y_stride]
    long long y_stride;
    const void* w;               // [channels, taps]
    const void* b;               // [channels] or null
    uint8_t* state;
    long long state_stride, state_offset;
    const int* token_seq;
    const int* q_start;
    const int* slot_ids;
    int rows, channels, taps, silu;
};

template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_kernel(ConvArgs a) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int row = blockIdx.y;
    if (c >= a.channels) return;
    const int seq = a.token_seq[row];
    if (seq < 0) return;
    const int o = row - a.q_start[seq];
    const float* st = (const float*)(a.state + (size_t)a.slot_ids[seq] * a.state_stride + a.state_offset);
    float acc = a.b ? to_f32(((const T*)a.b)[c]) : 0.f;
    for (int j = 0; j < a.taps; ++j) {
        const int back = a.taps - 1 - j;
        float xv;
        if (o - back >= 0) xv = to_f32(((const T*)a.x)[(size_t)(row - back) * a.x_stride + c]);
        else xv = st[(size_t)(a.taps - 1 + (o - back)) * a.channels + c];
        acc = fmaf(to_f32(((const T*)a.w)[(size_t)c * a.taps + j]), xv, acc);
    }
    if (a.silu) acc = silu_f32(acc);
    ((T*)a.y)[(size_t)row * a.y_stride + c] = from_f32<T>(acc);
}

#define CONV_ROWS_PER_THREAD 4
// The same with 16 bytes of neighbouring channels and four neighbouring rows a thread (8 bfloat16 or 4 float32 numbers): for rows and channel
// counts that allow aligned loads.  The thread's weights (its channels' TAPS numbers each lie one after the other)
// and biases come as 16-byte loads too: loaded one by one, lanes 64 bytes apart, they cost sixteen cache lines an
// instruction and the kernel five times its time.
template <typename T, int TAPS>
__global__ void __launch_bounds__(128)
causal_conv_vec_kernel(ConvArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int VEC = 16 / sizeof(T), RPT = CONV_ROWS_PER_THREAD, SPAN = RPT + TAPS - 1;
    const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    const int row0 = blockIdx.y * RPT;
    if (c0 >= a.channels) return;
    T wl[VEC * TAPS], bl[VEC];
#pragma unroll
    for (int u = 0; u < TAPS; ++u)
        *reinterpret_cast<uint4*>(wl + u * VEC) = *reinterpret_cast<const uint4*>((const T*)a.w + (size_t)c0 * TAPS + u * VEC);
    if (a.b) *reinterpret_cast<uint4*>(bl) = *reinterpret_cast<const uint4*>((const T*)a.b + c0);
    // the RPT rows of this thread and the TAPS - 1 rows before them, loaded once: a row serves up to TAPS outputs
    T xin[SPAN][VEC];
#pragma unroll
    for (int u = 0; u < SPAN; ++u) {
        const int r = row0 - (TAPS - 1) + u;
        if (r >= 0 && r < a.rows) *reinterpret_cast<uint4*>(xin[u]) = *reinterpret_cast<const uint4*>((const T*)a.x + (size_t)r * a.x_stride + c0);
    }
#pragma unroll
    for (int rr = 0; rr < RPT; ++rr) {
        const int row = row0 + rr;
        if (row >= a.rows) break;
        const int seq = a.token_seq[row];
        if (seq < 0) continue;
        const int o = row - a.q_start[seq];
        const float* st = (const float*)(a.state + (size_t)a.slot_ids[seq] * a.state_stride + a.state_offset);
        float acc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = a.b ? to_f32(bl[e]) : 0.f;
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
            const int back = TAPS - 1 - j;
            float xv[VEC];
            if (o - back >= 0) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) xv[e] = to_f32(xin[rr + j][e]);       // row - back = row0 - (TAPS - 1) + rr + j
            } else {
                const float* sp = st + (size_t)(TAPS - 1 + (o - back)) * a.channels + c0;
#pragma unroll
                for (int e = 0; e < VEC; ++e) xv[e] = sp[e];
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[e] = fmaf(to_f32(wl[e * TAPS + j]), xv[e], acc[e]);
        }
        T out[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) out[e] = from_f32<T>(a.silu ? silu_f32(acc[e]) : acc[e]);
        *reinterpret_cast<uint4*>((T*)a.y + (size_t)row * a.y_stride + c0) = *reinterpret_cast<const uint4*>(out);
    }
}

// The state after the step: the sequence's last taps - 1 inputs.  One thread per (sequence, channel)
// reads what it needs of the old state before it writes (entry i takes old entry i + n, n the step's
// tokens of the sequence, or a row of the step), in rising i: no other thread touches its column.
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_kernel(ConvArgs a, const int* __restrict__ q_len, int n_seqs) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.y;
    if (c >= a.channels || seq >= n_seqs) return;
    const int n = q_len[seq], r0 = a.q_start[seq];
    float* st = (float*)(a.state + (size_t)a.slot_ids[seq] * a.state_stride + a.state_offset);
    const int keep = a.taps - 1;
    for (int i = 0; i < keep; ++i) {
        const int o = n - keep + i;                  // the step's token that entry i holds, if not negative
        float v;
        if (o >= 0) v = to_f32(((const T*)a.x)[(size_t)(r0 + o) * a.x_stride + c]);
        else v = st[(size_t)(i + n) * a.channels + c];
        st[(size_t)i * a.channels + c] = v;
    }
}

extern "C" int braid_causal_conv(const void* x, long long x_stride, void* y, long long y_stride, const void* w, const void* b,
                                 int dtype, void* state, long long state_stride, long long state_offset,
                                 const int* token_seq, const int* q_start, const int* q_len, const int* slot_ids,
                                 int rows, int n_seqs, int channels, int taps, int silu, void* stream) {
    if (rows <= 0 || n_seqs <= 0) return BRAID_OK;
    if (channels <= 0 || taps < 1) BRAID_REFUSE("causal_conv: channels=%d and taps=%d must be positive", channels, taps);
    if (!state || (state_offset & 3) || (state_stride & 3)) BRAID_REFUSE("causal_conv: the state area must be given, in multiples of 4 bytes");
    if (rows > 65535 * 16 || n_seqs > 65535) BRAID_REFUSE("causal_conv: the step exceeds the grid limits");
    ConvArgs a{x, x_stride, y, y_stride, w, b, (uint8_t*)state, state_stride, state_offset, token_seq, q_start, slot_ids,
               rows, channels, taps, silu};
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    dim3 g1((channels + threads - 1) / threads, rows), g2((channels + threads - 1) / threads, n_seqs);
    if (g1.y > 65535) BRAID_REFUSE("causal_conv: %d rows exceed one launch", rows);
    if (dtype != BRAID_F32 && dtype != BRAID_BF16) BRAID_REFUSE("causal_conv: unknown dtype code %d", dtype);
    const int vec = dtype == BRAID_F32 ? 4 : 8;
    const bool wide = taps >= 2 && taps <= 4 && channels % vec == 0 && x_stride % vec == 0 && y_stride % vec == 0 &&
                      (((uintptr_t)x | (uintptr_t)y | (uintptr_t)w | (uintptr_t)b) & 15) == 0;
    const dim3 gv((channels / vec + 127) / 128, (rows + CONV_ROWS_PER_THREAD - 1) / CONV_ROWS_PER_THREAD);
#define CONV_LAUNCH(TT)                                                                                       \
    do {                                                                                                      \
        if (wide && taps == 2) braid_launch(causal_conv_vec_kernel<TT, 2>, gv, dim3(128), 0, s, a);           \
        else if (wide && taps == 3) braid_launch(causal_conv_vec_kernel<TT, 3>, gv, dim3(128), 0, s, a);      \
        else if (wide) braid_launch(causal_conv_vec_kernel<TT, 4>, gv, dim3(128), 0, s, a);                   \
        else braid_launch(causal_conv_kernel<TT>, g1, dim3(threads), 0, s, a);                                \
        if (taps > 1) braid_launch(conv_state_kernel<TT>, g2, dim3(threads), 0, s, a, q_len, n_seqs);         \
    } while (0)
    if (dtype == BRAID_F32) CONV_LAUNCH(float);
    else CONV_LAUNCH(__nv_bfloat16);
#undef CONV_LAUNCH
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ the linear recurrence
// Per sequence and head, token by token:  S <- diag(a_t) S + (kappa_t k_t) v_t^T,  o_t = S^T (q_scale q_t) + skip * v_t.
// S is [dk, dv] float32 in the sequence's state.
//   DECAY_CHANNEL (gated linear attention): a_t[i] = sigmoid(z_t[h, i] + zb[h, i])^(1 / tau), kappa = 1, no skip;
//       z float32 [rows, heads * dk].
//   DECAY_HEAD (state-space duality): dt = softplus(d_t[h] + dt_bias[h]), a_t = exp(-exp(A_log[h]) dt) for every
//       channel, kappa = dt, skip = D[h]; d in the run's type [rows, heads] (row stride gate_stride).
//   DECAY_GIVEN (a matrix memory whose gates were worked out before, braid_mlstm_gates): a_t = gate[t, h] for every
//       channel and kappa_t = kappa[t, h], both float32 with row stride gate_stride; no skip.  With `v_cols` < dv the
//       value columns from v_cols on read as 1: the state's column v_cols is then the sum of the decayed keys
//       (a normaliser), and the output's column v_cols its product with the query.
// q and k: [rows, groups, dk] in the run's type (head h reads group h / (heads / groups)); v: [rows, heads, dv].
// out: float32 [rows, heads * dv].  Everything is float32 arithmetic on the ordinary pipes: the recurrence, its
// decays and its state are not to be rounded to fewer bits.
//
// A CTA of 128 threads owns (head, sequence, a tile of value columns); a thread keeps a tile of R rows x 4 columns
// of S in registers (R = 8, or 16 for key sizes above 128); the RG row groups (R RG >= dk, RG a power of two up to
// 16) of a column group lie in one warp, so that a column's partial sums meet by warp shuffles, and two
// neighbouring lanes hold neighbouring column groups, so that a pair's loads and stores of S fill whole 32-byte
// sectors.  Tokens are staged SCAN_TB at a time in shared memory (q, k, the decays, v), read back 16 bytes at a
// time, and the walk has no block-wide barrier per token.
//
// Long prompts: a walk token by token is a chain as long as the prompt, on few CTAs.  For those the sequence is cut
// into chunks of `chunk` tokens that run side by side, in three passes over the same arithmetic:
//   pass 1  every chunk from a zero state: its own contribution U_c and the product D_c of its decays
//   carry   per state element, chunk after chunk: S_c (the state a chunk starts from) is kept, S <- D_c S + U_c
//   pass 3  every chunk from S_c, writing the outputs
// The sums are the sequential ones regrouped (D (S) + U instead of a step at a time), so results differ from the
// one-pass walk by rounding only.  Twice the arithmetic, a chain of 2 x chunk tokens, chunks x as many CTAs.
#define SCAN_CV 4
#define SCAN_THREADS 128
#define SCAN_TB 8
#define SCAN_MAX_DK 256
#define DECAY_CHANNEL 0
#define DECAY_HEAD 1
#define DECAY_GIVEN 2

struct ScanArgs {
    const void* q; long long q_stride;
    const void* k; long long k_stride;
    const void* v; long long v_stride;
    const void* gate; long long gate_stride;   // z (float32) or d (run type)
    const void* gate_bias;       // zb [heads * dk] or dt_bias [heads], run type
    const void* a_log;           // [heads], run type (DECAY_HEAD)
    const void* skip;            // [heads], run type, or null
    float* out; long long out_stride;
    uint8_t* state; long long state_stride, state_offset;
    const int* q_start; const int* q_len; const int* slot_ids;
    int heads, groups, dk, dv;
    float q_scale, inv_tau;
    // chunked walk (pass != 0): wbuf [seq][chunk][head][dk][dv], dbuf [seq][chunk][head]([dk])
    float* wbuf; float* dbuf;
    int pass, chunk, max_chunks;
    int gate_is_decay;           // DECAY_CHANNEL: `gate` holds the decays themselves (braid_scan_decay), not their logits
    const float* kappa;          // DECAY_GIVEN: the factor on the key, [rows, heads] with row stride gate_stride
    int v_cols;                  // columns a head that v really holds (row stride v_stride); the rest of dv read as 1
};

// sigmoid(z)^(1 / tau) through log sigmoid(z) = min(z, 0) - log1p(exp(-|z|)): no overflow, full precision near one
__device__ __forceinline__ float decay_of_logit(float z, float inv_tau) {
    return expf((fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) * inv_tau);
}

// z[r, c] <- sigmoid(z[r, c] + b[c])^(1 / tau) in place: the decays of a long step, computed once instead of by every
// CTA that walks a tile of the head's value columns, in every pass.
template <typename T>
__global__ void scan_decay_kernel(float* __restrict__ z, long long stride, const T* __restrict__ b, long long total, int n, float inv_tau) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / n;
    const int c = (int)(i - r * n);
    z[r * stride + c] = decay_of_logit(z[r * stride + c] + to_f32(b[c]), inv_tau);
}

extern "C" int braid_scan_decay(float* z, long long stride, const void* bias, int dtype, int rows, int n, float inv_tau, void* stream) {
    if (rows <= 0 || n <= 0) return BRAID_OK;
    const long long total = (long long)rows * n;
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("scan_decay: %lld elements exceed one launch", total);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32) braid_launch(scan_decay_kernel<float>, dim3((int)blocks), dim3(256), 0, s, z, stride, (const float*)bias, total, n, inv_tau);
    else if (dtype == BRAID_BF16) braid_launch(scan_decay_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, s, z, stride, (const __nv_bfloat16*)bias, total, n, inv_tau);
    else BRAID_REFUSE("scan_decay: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

template <typename T, int MODE, int RG, int R>
__global__ void __launch_bounds__(SCAN_THREADS)
linear_scan_kernel(ScanArgs a) {
    constexpr int CV = SCAN_CV, CG = SCAN_THREADS / RG, DVT = CG * CV, DKP = RG * R;
    constexpr int TB = DKP <= 128 ? SCAN_TB : SCAN_TB / 2;      // tokens a batch: what a thread holds of the next batch fits its registers
    static_assert(RG >= 2 && RG <= 16 && (R == 8 || R == 16), "two column groups and RG row groups share a warp");
    static_assert((TB * DKP) % SCAN_THREADS == 0 && (TB * DVT) % SCAN_THREADS == 0, "a batch is a whole number of elements a thread");
    pdl_trigger();
    const int h = blockIdx.x, seq = blockIdx.y;
    const int n_dvt = (a.dv + DVT - 1) / DVT;
    const int dvt = blockIdx.z % n_dvt, c = blockIdx.z / n_dvt;
    const int tid = threadIdx.x;
    // lane bit 0: the lower bit of the column group; the next bits: the row group; what is left: the column group's rest
    const int rg = (tid >> 1) % RG, cg = (tid & 1) | ((tid / (2 * RG)) << 1);
    const int j0 = dvt * DVT + cg * CV;
    const int n = a.q_len[seq], r0 = a.q_start[seq];
    int t_begin = 0, t_end = n;
    if (a.pass != 0) { t_begin = c * a.chunk; t_end = min(n, t_begin + a.chunk); }
    if (t_begin >= t_end) return;
    const int dk = a.dk, dv = a.dv;
    const int g = h / (a.heads / a.groups);
    extern __shared__ __align__(16) float sm[];
    float* sq = sm;                                          // [TB][DKP]
    float* sk = sq + TB * DKP;
    float* sv = sk + TB * DKP;                               // [TB][DVT]
    float* skap = sv + TB * DVT;                             // [TB] step sizes, [TB] decays of the head (8 floats each)
    float* sah = skap + SCAN_TB;
    float* sa = sah + SCAN_TB;                               // [TB][DKP] decays per channel (DECAY_CHANNEL)
    float head_a = 0.f, head_bias = 0.f, head_skip = 0.f;
    if (MODE == DECAY_HEAD) {
        head_a = -expf(to_f32(((const T*)a.a_log)[h]));
        head_bias = to_f32(((const T*)a.gate_bias)[h]);
        if (a.skip) head_skip = to_f32(((const T*)a.skip)[h]);
    }
    pdl_wait();
    const size_t per_head = (size_t)dk * dv;
    float* S_area = (float*)(a.state + (size_t)a.slot_ids[seq] * a.state_stride + a.state_offset) + (size_t)h * per_head;
    float* S_work = a.wbuf ? a.wbuf + ((size_t)(seq * a.max_chunks + c) * a.heads + h) * per_head : nullptr;
    float s[R][CV];
#pragma unroll
    for (int e = 0; e < R; ++e)
#pragma unroll
        for (int x = 0; x < CV; ++x) {
            const int i = rg * R + e, j = j0 + x;
            s[e][x] = (a.pass != 1 && i < dk && j < dv) ? (a.pass == 0 ? S_area : S_work)[(size_t)i * dv + j] : 0.f;
        }
    float dprod[R];
#pragma unroll
    for (int e = 0; e < R; ++e) dprod[e] = 1.f;
    float hprod = 1.f;
    const bool outputs = a.pass != 1;

    // A batch of TB tokens is asked for from global memory while the batch before it is walked: its numbers wait in
    // registers (as they came, in the run's type) and go to shared memory, converted, when the walk has left it.
    constexpr int NQ = TB * DKP / SCAN_THREADS, NV = TB * DVT / SCAN_THREADS;
    T pq[NQ], pk[NQ], pv[NV], pg = from_f32<T>(0.f);
    float pgd = 0.f, pgk = 0.f;
    float pa[MODE == DECAY_CHANNEL ? NQ : 1];
    auto fetch = [&](int t0) {
        const int nt = min(TB, t_end - t0);
#pragma unroll
        for (int u = 0; u < NQ; ++u) {
            const int idx = tid + u * SCAN_THREADS;
            const int t = idx / DKP, i = idx - t * DKP;
            const size_t row = (size_t)(r0 + t0 + t);
            const bool in = t < nt && i < dk;
            pq[u] = in ? ((const T*)a.q)[row * a.q_stride + (size_t)g * dk + i] : from_f32<T>(0.f);
            pk[u] = in ? ((const T*)a.k)[row * a.k_stride + (size_t)g * dk + i] : from_f32<T>(0.f);
            if (MODE == DECAY_CHANNEL) pa[u] = in ? ((const float*)a.gate)[row * a.gate_stride + (size_t)h * dk + i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < NV; ++u) {
            const int idx = tid + u * SCAN_THREADS;
            const int t = idx / DVT, jj = idx - t * DVT;
            const size_t row = (size_t)(r0 + t0 + t);
            const int col = dvt * DVT + jj;
            pv[u] = (t < nt && col < a.v_cols) ? ((const T*)a.v)[row * a.v_stride + (size_t)h * a.v_cols + col]
                                              : from_f32<T>((t < nt && col < dv) ? 1.f : 0.f);
        }
        if (MODE == DECAY_HEAD && tid < nt) pg = ((const T*)a.gate)[(size_t)(r0 + t0 + tid) * a.gate_stride + h];
        if (MODE == DECAY_GIVEN && tid < nt) {
            pgd = ((const float*)a.gate)[(size_t)(r0 + t0 + tid) * a.gate_stride + h];
            pgk = a.kappa[(size_t)(r0 + t0 + tid) * a.gate_stride + h];
        }
    };
    fetch(t_begin);
    for (int t0 = t_begin; t0 < t_end; t0 += TB) {
        const int nt = min(TB, t_end - t0);
        __syncthreads();                                    // the batch before has been read
#pragma unroll
        for (int u = 0; u < NQ; ++u) {
            const int idx = tid + u * SCAN_THREADS;
            sq[idx] = to_f32(pq[u]) * a.q_scale;
            sk[idx] = to_f32(pk[u]);
            if (MODE == DECAY_CHANNEL) {
                float av = pa[u];
                if (!a.gate_is_decay) {
                    const int i = idx % DKP;
                    av = i < dk ? decay_of_logit(av + to_f32(((const T*)a.gate_bias)[(size_t)h * dk + i]), a.inv_tau) : 0.f;
                }
                sa[idx] = av;
            }
        }
#pragma unroll
        for (int u = 0; u < NV; ++u) sv[tid + u * SCAN_THREADS] = to_f32(pv[u]);
        if (MODE == DECAY_HEAD && tid < nt) {
            const float x = to_f32(pg) + head_bias;
            const float dt = x > 20.f ? x : log1pf(expf(x));           // softplus
            skap[tid] = dt;
            sah[tid] = expf(head_a * dt);
        }
        if (MODE == DECAY_GIVEN && tid < nt) { skap[tid] = pgk; sah[tid] = pgd; }
        if (t0 + TB < t_end) fetch(t0 + TB);
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            float qv[R], kv[R], av[R], vv[CV];
#pragma unroll
            for (int e = 0; e < R; e += 4)
                *reinterpret_cast<float4*>(kv + e) = *reinterpret_cast<const float4*>(sk + t * DKP + rg * R + e);
            *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(sv + t * DVT + cg * CV);
            if (MODE == DECAY_CHANNEL) {
#pragma unroll
                for (int e = 0; e < R; e += 4)
                    *reinterpret_cast<float4*>(av + e) = *reinterpret_cast<const float4*>(sa + t * DKP + rg * R + e);
            } else {
                const float ah = sah[t], kap = skap[t];
                hprod *= ah;
#pragma unroll
                for (int e = 0; e < R; ++e) { av[e] = ah; kv[e] *= kap; }
            }
#pragma unroll
            for (int e = 0; e < R; ++e) {
                dprod[e] *= av[e];
#pragma unroll
                for (int x = 0; x < CV; ++x) s[e][x] = fmaf(av[e], s[e][x], kv[e] * vv[x]);
            }
            if (outputs) {
#pragma unroll
                for (int e = 0; e < R; e += 4)
                    *reinterpret_cast<float4*>(qv + e) = *reinterpret_cast<const float4*>(sq + t * DKP + rg * R + e);
                float acc[CV];
#pragma unroll
                for (int x = 0; x < CV; ++x) acc[x] = 0.f;
#pragma unroll
                for (int e = 0; e < R; ++e)
#pragma unroll
                    for (int x = 0; x < CV; ++x) acc[x] = fmaf(s[e][x], qv[e], acc[x]);
#pragma unroll
                for (int o = RG; o >= 2; o >>= 1)          // the row groups are lane bits 1 ...
#pragma unroll
                    for (int x = 0; x < CV; ++x) acc[x] += __shfl_xor_sync(0xffffffffu, acc[x], o);
                if (rg == 0) {
                    float* orow = a.out + (size_t)(r0 + t0 + t) * a.out_stride + (size_t)h * dv;
#pragma unroll
                    for (int x = 0; x < CV; ++x)
                        if (j0 + x < dv) orow[j0 + x] = acc[x] + head_skip * vv[x];
                }
            }
        }
    }
    if (a.pass == 3) return;
    float* dst = a.pass == 0 ? S_area : S_work;
#pragma unroll
    for (int e = 0; e < R; ++e)
#pragma unroll
        for (int x = 0; x < CV; ++x) {
            const int i = rg * R + e, j = j0 + x;
            if (i < dk && j < dv) dst[(size_t)i * dv + j] = s[e][x];
        }
    if (a.pass == 1 && dvt == 0) {                           // the product of the chunk's decays, once per head
        const size_t base = (size_t)(seq * a.max_chunks + c) * a.heads + h;
        if (MODE != DECAY_CHANNEL) {
            if (tid == 0) a.dbuf[base] = hprod;
        } else if (cg == 0) {
#pragma unroll
            for (int e = 0; e < R; ++e)
                if (rg * R + e < dk) a.dbuf[base * dk + rg * R + e] = dprod[e];
        }
    }
}

// The carry between the chunks of a sequence: per element of the state, chunk after chunk.
template <int MODE>
__global__ void __launch_bounds__(256)
scan_carry_kernel(ScanArgs a) {
    pdl_trigger();
    pdl_wait();
    const size_t per_seq = (size_t)a.heads * a.dk * a.dv;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.y;
    if (idx >= per_seq) return;
    const int n = a.q_len[seq];
    if (n <= 0) return;
    const int n_chunks = (n + a.chunk - 1) / a.chunk;
    const int h = (int)(idx / ((size_t)a.dk * a.dv));
    const int i = (int)((idx / a.dv) % a.dk);
    float* S_area = (float*)(a.state + (size_t)a.slot_ids[seq] * a.state_stride + a.state_offset);
    float S = S_area[idx];
    for (int c = 0; c < n_chunks; ++c) {
        const size_t base = (size_t)(seq * a.max_chunks + c);
        float* w = a.wbuf + base * per_seq + idx;
        const float u = *w;
        const float d = MODE != DECAY_CHANNEL ? a.dbuf[base * a.heads + h] : a.dbuf[(base * a.heads + h) * a.dk + i];
        *w = S;                                             // the state that chunk c starts from
        S = fmaf(d, S, u);
    }
    S_area[idx] = S;
}

static int scan_rg(int dk) { return dk <= 32 ? 4 : dk <= 64 ? 8 : 16; }
static int scan_rows(int dk) { return dk <= 128 ? 8 : 16; }

// Floats of scratch that the chunked walk of a step needs (0: the step is walked in one pass).
extern "C" long long braid_linear_scan_work_floats(int n_seqs, int max_q_len, int chunk, int heads, int dk, int dv, int mode) {
    if (chunk <= 0 || max_q_len < 2 * chunk) return 0;
    const long long chunks = (max_q_len + chunk - 1) / chunk;
    return (long long)n_seqs * chunks * heads * ((long long)dk * dv + (mode != DECAY_CHANNEL ? 1 : dk));
}

extern "C" int braid_linear_scan(const void* q, long long q_stride, const void* k, long long k_stride, const void* v,
                                 long long v_stride, const void* gate, long long gate_stride, const void* gate_bias,
                                 const void* a_log, const void* skip, float* out, long long out_stride, void* state,
                                 long long state_stride, long long state_offset, const int* q_start, const int* q_len,
                                 const int* slot_ids, int dtype, int mode, int n_seqs, int heads, int groups, int dk, int dv,
                                 float q_scale, float inv_tau, int max_q_len, int chunk, float* work, long long work_floats,
                                 int gate_is_decay, const float* kappa, int v_cols, void* stream) {
    if (n_seqs <= 0) return BRAID_OK;
    if (heads <= 0 || groups <= 0 || heads % groups) BRAID_REFUSE("linear_scan: %d heads do not divide into %d groups", heads, groups);
    if (dk <= 0 || dk > SCAN_MAX_DK || dv <= 0) BRAID_REFUSE("linear_scan: key size %d must be in (0, %d], value size %d positive", dk, SCAN_MAX_DK, dv);
    if (!state || (state_offset & 3) || (state_stride & 3)) BRAID_REFUSE("linear_scan: the state area must be given, in multiples of 4 bytes");
    if (mode != DECAY_CHANNEL && mode != DECAY_HEAD && mode != DECAY_GIVEN) BRAID_REFUSE("linear_scan: unknown decay mode %d", mode);
    if (mode == DECAY_GIVEN && !kappa) BRAID_REFUSE("linear_scan: given decays come with the factors on the keys");
    if (v_cols <= 0 || v_cols > dv) v_cols = dv;
    if (mode != DECAY_GIVEN && v_cols != dv) BRAID_REFUSE("linear_scan: value columns that read as 1 need given decays");
    if (mode == DECAY_HEAD && !a_log) BRAID_REFUSE("linear_scan: a decay per head needs A_log");
    if (dtype != BRAID_F32 && dtype != BRAID_BF16) BRAID_REFUSE("linear_scan: unknown dtype code %d", dtype);
    const int rg = scan_rg(dk), rr = scan_rows(dk);
    const int dvt = (SCAN_THREADS / rg) * SCAN_CV;
    const int n_dvt = (dv + dvt - 1) / dvt;
    const long long need = braid_linear_scan_work_floats(n_seqs, max_q_len, chunk, heads, dk, dv, mode);
    const bool chunked = need > 0 && work != nullptr;
    if (chunked && need > work_floats) BRAID_REFUSE("linear_scan: the chunked walk needs %lld floats of scratch, it was given %lld", need, work_floats);
    const int max_chunks = chunked ? (max_q_len + chunk - 1) / chunk : 1;
    if (n_seqs > 65535 || (long long)n_dvt * max_chunks > 65535) BRAID_REFUSE("linear_scan: the step exceeds the grid limits");
    ScanArgs a{q, q_stride, k, k_stride, v, v_stride, gate, gate_stride, gate_bias, a_log, skip, out, out_stride,
               (uint8_t*)state, state_stride, state_offset, q_start, q_len, slot_ids, heads, groups, dk, dv, q_scale, inv_tau,
               nullptr, nullptr, 0, chunk, max_chunks, gate_is_decay, kappa, v_cols};
    if (chunked) {
        a.wbuf = work;
        a.dbuf = work + (long long)n_seqs * max_chunks * heads * dk * dv;
    }
    const size_t smem = (size_t)(SCAN_TB * (2 * rg * rr + dvt + 2) + (mode == DECAY_CHANNEL ? SCAN_TB * rg * rr : 0)) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 block(SCAN_THREADS);
#define SCAN_LAUNCH_RG(TT, MM, GRID)                                                                          \
    do {                                                                                                      \
        if (rg == 4) braid_launch(linear_scan_kernel<TT, MM, 4, 8>, GRID, block, smem, s, a);                 \
        else if (rg == 8) braid_launch(linear_scan_kernel<TT, MM, 8, 8>, GRID, block, smem, s, a);            \
        else if (rr == 8) braid_launch(linear_scan_kernel<TT, MM, 16, 8>, GRID, block, smem, s, a);           \
        else braid_launch(linear_scan_kernel<TT, MM, 16, 16>, GRID, block, smem, s, a);                       \
    } while (0)
#define SCAN_LAUNCH(GRID)                                                                                     \
    do {                                                                                                      \
        if (dtype == BRAID_F32 && mode == DECAY_CHANNEL) SCAN_LAUNCH_RG(float, DECAY_CHANNEL, GRID);          \
        else if (dtype == BRAID_F32 && mode == DECAY_HEAD) SCAN_LAUNCH_RG(float, DECAY_HEAD, GRID);           \
        else if (dtype == BRAID_F32) SCAN_LAUNCH_RG(float, DECAY_GIVEN, GRID);                                \
        else if (mode == DECAY_CHANNEL) SCAN_LAUNCH_RG(__nv_bfloat16, DECAY_CHANNEL, GRID);                   \
        else if (mode == DECAY_HEAD) SCAN_LAUNCH_RG(__nv_bfloat16, DECAY_HEAD, GRID);                         \
        else SCAN_LAUNCH_RG(__nv_bfloat16, DECAY_GIVEN, GRID);                                                \
    } while (0)
    if (!chunked) {
        const dim3 grid(heads, n_seqs, n_dvt);
        SCAN_LAUNCH(grid);
        BRAID_LAUNCH_CHECK();
    }
    const dim3 grid(heads, n_seqs, n_dvt * max_chunks);
    a.pass = 1;
    SCAN_LAUNCH(grid);
    const long long per_seq = (long long)heads * dk * dv;
    const dim3 cgrid((unsigned)((per_seq + 255) / 256), n_seqs);
    if (mode != DECAY_CHANNEL) braid_launch(scan_carry_kernel<DECAY_HEAD>, cgrid, dim3(256), 0, s, a);
    else braid_launch(scan_carry_kernel<DECAY_CHANNEL>, cgrid, dim3(256), 0, s, a);
    a.pass = 3;
    SCAN_LAUNCH(grid);
#undef SCAN_LAUNCH
#undef SCAN_LAUNCH_RG
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ gated RMS norm
// y [rows, width] float32 (a recurrence's output), gate [rows, gate_stride] in the run's type, in groups of `group`
// columns, each normed by its own root mean square:
//   gate_first = 0:  out = y / rms(y) * w * silu(gate) * out_scale         (norm, then gate)
//   gate_first = 1:  u = y * silu(gate);  out = u / rms(u) * w * out_scale (gate, then norm)
// w has w_len numbers; column c of the row reads w[c % w_len] (w_len = group: one weight for every group;
// w_len = width: a weight per column).  One warp per (row, group).  Everything in float32; out in the run's type.
template <typename T>
__global__ void __launch_bounds__(128)
gated_norm_kernel(const float* __restrict__ y, const T* __restrict__ gate, long long gate_stride, const T* __restrict__ w,
                  int w_len, T* __restrict__ out, long long out_stride, const int* __restrict__ token_seq, int rows,
                  int width, int group, int gate_first, float eps, float out_scale) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups = width / group;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)rows * groups) return;
    const int row = (int)(item / groups), gi = (int)(item - (long long)row * groups);
    if (token_seq[row] < 0) return;
    const float* yr = y + (size_t)row * width + (size_t)gi * group;
    const T* gr = gate + (size_t)row * gate_stride + (size_t)gi * group;
    float ss = 0.f;
    for (int c = lane; c < group; c += 32) {
        float u = yr[c];
        if (gate_first) u *= silu_f32(to_f32(gr[c]));
        ss = fmaf(u, u, ss);
    }
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)group + eps);
    T* orow = out + (size_t)row * out_stride + (size_t)gi * group;
    for (int c = lane; c < group; c += 32) {
        const float sg = silu_f32(to_f32(gr[c]));
        const float wv = to_f32(w[(gi * group + c) % w_len]);
        float u = yr[c];
        u = gate_first ? (u * sg) * r * wv : (u * r * wv) * sg;
        orow[c] = from_f32<T>(u * out_scale);
    }
}

// The same with a CTA of 128 threads a (row, group): for groups of more than 128 columns, where a warp alone would
// walk a long way (a decode step of 8 rows and 8 groups of 512 columns: 21 -> 11.5 us).
template <typename T>
__global__ void __launch_bounds__(128)
gated_norm_block_kernel(const float* __restrict__ y, const T* __restrict__ gate, long long gate_stride, const T* __restrict__ w,
                        int w_len, T* __restrict__ out, long long out_stride, const int* __restrict__ token_seq, int rows,
                        int width, int group, int gate_first, float eps, float out_scale) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int groups = width / group;
    const int row = blockIdx.x / groups, gi = blockIdx.x - row * groups;
    if (token_seq[row] < 0) return;
    const float* yr = y + (size_t)row * width + (size_t)gi * group;
    const T* gr = gate + (size_t)row * gate_stride + (size_t)gi * group;
    float ss = 0.f;
    for (int c = threadIdx.x; c < group; c += blockDim.x) {
        float u = yr[c];
        if (gate_first) u *= silu_f32(to_f32(gr[c]));
        ss = fmaf(u, u, ss);
    }
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)group + eps);
    T* orow = out + (size_t)row * out_stride + (size_t)gi * group;
    for (int c = threadIdx.x; c < group; c += blockDim.x) {
        const float sg = silu_f32(to_f32(gr[c]));
        const float wv = to_f32(w[(gi * group + c) % w_len]);
        float u = yr[c];
        u = gate_first ? (u * sg) * r * wv : (u * r * wv) * sg;
        orow[c] = from_f32<T>(u * out_scale);
    }
}

extern "C" int braid_gated_norm(const float* y, const void* gate, long long gate_stride, const void* w, int w_len, void* out,
                                long long out_stride, const int* token_seq, int dtype, int rows, int width, int group,
                                int gate_first, float eps, float out_scale, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (width <= 0 || group <= 0 || width % group) BRAID_REFUSE("gated_norm: width %d is not a whole number of groups of %d", width, group);
    if (w_len <= 0) BRAID_REFUSE("gated_norm: the weight has no numbers");
    const long long items = (long long)rows * (width / group);
    const long long blocks = (items + 3) / 4;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("gated_norm: %lld (row, group) pairs exceed one launch", items);
    cudaStream_t s = (cudaStream_t)stream;
    if (group > 128 && items <= 0x7fffffffLL) {
        if (dtype == BRAID_F32)
            braid_launch(gated_norm_block_kernel<float>, dim3((int)items), dim3(128), 0, s, y, (const float*)gate, gate_stride,
                         (const float*)w, w_len, (float*)out, out_stride, token_seq, rows, width, group, gate_first, eps, out_scale);
        else if (dtype == BRAID_BF16)
            braid_launch(gated_norm_block_kernel<__nv_bfloat16>, dim3((int)items), dim3(128), 0, s, y, (const __nv_bfloat16*)gate,
                         gate_stride, (const __nv_bfloat16*)w, w_len, (__nv_bfloat16*)out, out_stride, token_seq, rows, width, group,
                         gate_first, eps, out_scale);
        else BRAID_REFUSE("gated_norm: unknown dtype code %d", dtype);
        BRAID_LAUNCH_CHECK();
    }
    if (dtype == BRAID_F32)
        braid_launch(gated_norm_kernel<float>, dim3((int)blocks), dim3(128), 0, s, y, (const float*)gate, gate_stride, (const float*)w,
                     w_len, (float*)out, out_stride, token_seq, rows, width, group, gate_first, eps, out_scale);
    else if (dtype == BRAID_BF16)
        braid_launch(gated_norm_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(128), 0, s, y, (const __nv_bfloat16*)gate, gate_stride,
                     (const __nv_bfloat16*)w, w_len, (__nv_bfloat16*)out, out_stride, token_seq, rows, width, group, gate_first, eps, out_scale);
    else BRAID_REFUSE("gated_norm: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ gates of a matrix memory (mLSTM)
// Per sequence and head, token by token, with a running maximum m that the state carries (float32 [heads] at
// state_offset; zero when a slot is taken, so m starts at 0):
//   li = cap tanh((zi + bi) / cap)                      log input gate
//   lf = log sigmoid(cap tanh((zf + bf) / cap))         log forget gate
//   m_t = max(lf + m_(t-1), li);  decay_t = exp(lf + m_(t-1) - m_t);  kappa_t = exp(li - m_t);  floor_t = exp(-m_t)
// z: float32 [rows, 2 heads] (the input gates' logits, then the forget gates'), biases [heads] each in the run's
// type.  out: float32 [rows, 3 heads]: decays, kappas, floors.  One warp a (sequence, head): a lane a token for
// the transcendental work; the chain over m is walked by every lane alike, so a token's m does not depend on where
// the step began.
template <typename T>
__global__ void __launch_bounds__(32)
mlstm_gates_kernel(const float* __restrict__ z, long long z_stride, const T* __restrict__ bi, const T* __restrict__ bf,
                   float* __restrict__ out, uint8_t* __restrict__ state, long long state_stride, long long state_offset,
                   const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ slot_ids,
                   int heads, float cap) {
    pdl_trigger();
    const int h = blockIdx.x, seq = blockIdx.y, lane = threadIdx.x;
    const float b_i = to_f32(bi[h]), b_f = to_f32(bf[h]);
    pdl_wait();
    const int n = q_len[seq], r0 = q_start[seq];
    if (n <= 0) return;
    float* mp = (float*)(state + (size_t)slot_ids[seq] * state_stride + state_offset) + h;
    float m = *mp;
    const float inv_cap = 1.f / cap;
    // the next 32 tokens' logits are asked for before this group's chain is walked, so the chain hides their way
    float zi_next = 0.f, zf_next = 0.f;
    if (lane < n) {
        const float* zr = z + (size_t)(r0 + lane) * z_stride;
        zi_next = zr[h];
        zf_next = zr[heads + h];
    }
    for (int t0 = 0; t0 < n; t0 += 32) {
        const int t = t0 + lane;
        const float zi = zi_next, zf = zf_next;
        if (t + 32 < n) {
            const float* zr = z + (size_t)(r0 + t + 32) * z_stride;
            zi_next = zr[h];
            zf_next = zr[heads + h];
        }
        float li = 0.f, lf = 0.f;
        if (t < n) {
            li = cap * tanhf((zi + b_i) * inv_cap);
            const float x = cap * tanhf((zf + b_f) * inv_cap);
            lf = fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
        }
        const int nt = min(32, n - t0);
        float m_prev = 0.f, m_mine = 0.f;
        if (nt == 32) {                      // a full group: unrolled, so the broadcasts run ahead of the chain
#pragma unroll
            for (int l = 0; l < 32; ++l) {
                const float f = __shfl_sync(0xffffffffu, lf, l), i = __shfl_sync(0xffffffffu, li, l);
                const float mn = fmaxf(f + m, i);
                if (l == lane) { m_prev = m; m_mine = mn; }
                m = mn;
            }
        } else {
            for (int l = 0; l < nt; ++l) {
                const float f = __shfl_sync(0xffffffffu, lf, l), i = __shfl_sync(0xffffffffu, li, l);
                const float mn = fmaxf(f + m, i);
                if (l == lane) { m_prev = m; m_mine = mn; }
                m = mn;
            }
        }
        if (t < n) {
            float* o = out + (size_t)(r0 + t) * (3 * heads);
            o[h] = expf(lf + m_prev - m_mine);
            o[heads + h] = expf(li - m_mine);
            o[2 * heads + h] = expf(-m_mine);
        }
    }
    if (lane == 0) *mp = m;
}

extern "C" int braid_mlstm_gates(const float* z, long long z_stride, const void* bi, const void* bf, int dtype, float* out,
                                 void* state, long long state_stride, long long state_offset, const int* q_start,
                                 const int* q_len, const int* slot_ids, int n_seqs, int heads, float cap, void* stream) {
    if (n_seqs <= 0) return BRAID_OK;
    if (heads <= 0 || n_seqs > 65535) BRAID_REFUSE("mlstm_gates: heads=%d must be positive and %d sequences fit a launch", heads, n_seqs);
    if (!(cap > 0.f)) BRAID_REFUSE("mlstm_gates: the cap %g must be positive", (double)cap);
    if (!state || (state_offset & 3) || (state_stride & 3)) BRAID_REFUSE("mlstm_gates: the state area must be given, in multiples of 4 bytes");
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(heads, n_seqs);
    if (dtype == BRAID_F32)
        braid_launch(mlstm_gates_kernel<float>, grid, dim3(32), 0, s, z, z_stride, (const float*)bi, (const float*)bf, out,
                     (uint8_t*)state, state_stride, state_offset, q_start, q_len, slot_ids, heads, cap);
    else if (dtype == BRAID_BF16)
        braid_launch(mlstm_gates_kernel<__nv_bfloat16>, grid, dim3(32), 0, s, z, z_stride, (const __nv_bfloat16*)bi,
                     (const __nv_bfloat16*)bf, out, (uint8_t*)state, state_stride, state_offset, q_start, q_len, slot_ids, heads, cap);
    else BRAID_REFUSE("mlstm_gates: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

// The memory's read-out: y [rows, heads * (dv + 1)] float32 holds, a head, S^T q in its first dv columns and n . q in
// the last.  o = y[:dv] / (max(|n . q|, floor) + 1e-6), floor = floors[row, head] (row stride floor_stride);
// out = o / sqrt(mean(o^2) + eps) * w[head * dv + c] * sigmoid(gate[row, head * dv + c]), in the run's type.
// One warp a (row, head); float32 throughout.
template <typename T>
__global__ void __launch_bounds__(128)
mlstm_out_kernel(const float* __restrict__ y, const float* __restrict__ floors, long long floor_stride,
                 const T* __restrict__ gate, long long gate_stride, const T* __restrict__ w, T* __restrict__ out,
                 long long out_stride, const int* __restrict__ token_seq, int rows, int heads, int dv, float eps) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)rows * heads) return;
    const int row = (int)(item / heads), h = (int)(item - (long long)row * heads);
    T* orow = out + (size_t)row * out_stride + (size_t)h * dv;
    if (token_seq[row] < 0) {
        for (int c = lane; c < dv; c += 32) orow[c] = from_f32<T>(0.f);
        return;
    }
    const float* yr = y + ((size_t)row * heads + h) * (dv + 1);
    const float inv = 1.f / (fmaxf(fabsf(yr[dv]), floors[(size_t)row * floor_stride + h]) + 1e-6f);
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) { const float u = yr[c] * inv; ss = fmaf(u, u, ss); }
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)dv + eps);
    const T* gr = gate + (size_t)row * gate_stride + (size_t)h * dv;
    for (int c = lane; c < dv; c += 32) {
        const float sg = 1.f / (1.f + expf(-to_f32(gr[c])));
        orow[c] = from_f32<T>(yr[c] * inv * r * to_f32(w[(size_t)h * dv + c]) * sg);
    }
}

extern "C" int braid_mlstm_out(const float* y, const float* floors, long long floor_stride, const void* gate,
                               long long gate_stride, const void* w, void* out, long long out_stride, const int* token_seq,
                               int dtype, int rows, int heads, int dv, float eps, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (heads <= 0 || dv <= 0) BRAID_REFUSE("mlstm_out: heads=%d and dv=%d must be positive", heads, dv);
    const long long blocks = ((long long)rows * heads + 3) / 4;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("mlstm_out: %lld (row, head) pairs exceed one launch", (long long)rows * heads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32)
        braid_launch(mlstm_out_kernel<float>, dim3((int)blocks), dim3(128), 0, s, y, floors, floor_stride, (const float*)gate,
                     gate_stride, (const float*)w, (float*)out, out_stride, token_seq, rows, heads, dv, eps);
    else if (dtype == BRAID_BF16)
        braid_launch(mlstm_out_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(128), 0, s, y, floors, floor_stride,
                     (const __nv_bfloat16*)gate, gate_stride, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_stride,
                     token_seq, rows, heads, dv, eps);
    else BRAID_REFUSE("mlstm_out: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}
