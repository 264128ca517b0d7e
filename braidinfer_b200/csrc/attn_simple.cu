// Plain attention over the paged cache: one warp per (token, query head).
//
// It is the float32 path's attention and the reference kernel that the faster
// bfloat16 kernels are checked against.  It serves prompts, chunks of prompts and
// single decoded tokens alike: every query reads its keys and values from the cache,
// which already holds the step's own tokens.
//
// Formula (kernels/megakernel_ops.hip:2192-2194, 2310-2342 of the reference): head h
// reads kv head h / g; s_j = (q . k_j) * scale; online softmax with running maximum m,
// denominator d and accumulator acc; out = acc / d.  Key j is visible to the query at
// position p iff j <= p and, with a window w > 0, p - j < w (the window is this
// library's own; the reference has none).  Scores, softmax and accumulation are float32.
// With has_sink (or head_sinks, a score a head), the denominator also counts one more term exp(sink_score) that has no value
// (an attention sink: p_j = exp(s_j) / (exp(sink_score) + sum_i exp(s_i))).  out_scale is a
// constant factor on the result.
// Options of other designs: keep_first > 0 lets every query also see the sequence's first keep_first positions
// whatever the window (visible: j <= p and (p - j < w or j < keep_first)); head_scale is a factor a head on the
// scores; value_heads > 1 applies a head's probabilities to the values of every kv head in turn (the item is then
// (token, query head, value head) and the result lies at virtual head `head * value_heads + value head`), which is
// what a mix of the heads' probabilities after the softmax needs (pointwise.cu, head_mix).
#include "common.cuh"

struct AttnSimpleArgs {
    const void* q;            // [rows, q_row_stride], head h at column h * hd
    void* out;                // [rows, out_row_stride]
    const void* cache;        // one layer: [page][2][nkh][page_size][hd]
    const int* page_table;    // [n_seqs, table_cols]
    const int* positions;     // [rows]
    const int* token_seq;     // [rows] or -1 for padding
    int q_row_stride, out_row_stride;
    int rows, nqh, nkh, hd, page_size, table_cols, num_pages, window;
    float scale;
    int has_sink;
    float sink_score, out_scale;
    int* error_flag;          // raised when a visible position has no page, or one outside the cache
    const float* head_sinks;  // [nqh] float32: a sink score a head (learned), instead of the one score; or null
    const void* head_gate;    // [rows, gate_stride] in the rows' type: the result of head h is multiplied by
    long long gate_stride;    // sigmoid(head_gate[row, h]); or null
    int keep_first;           // the first positions of a sequence stay visible beyond the window
    const float* head_scale;  // [nqh] float32: a factor a head on the scores; or null
    int value_heads;          // 1, or nkh: every query head reads the values of every kv head
};

#define ATTN_SIMPLE_WARPS 4
#define ATTN_SIMPLE_MAX_HD 256

template <typename T>
__global__ void __launch_bounds__(ATTN_SIMPLE_WARPS * 32)
attn_simple_kernel(AttnSimpleArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];                  // [warps][hd] queries, [warps][32] probabilities
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* qs = smem + warp * a.hd;
    float* ps = smem + ATTN_SIMPLE_WARPS * a.hd + warp * 32;
    const long long item = (long long)blockIdx.x * ATTN_SIMPLE_WARPS + warp;
    if (item >= (long long)a.rows * a.nqh * a.value_heads) return;
    const int row = (int)(item / (a.nqh * a.value_heads));
    const int vhead = (int)(item - (long long)row * a.nqh * a.value_heads);       // head * value_heads + value head
    const int head = vhead / a.value_heads;
    T* o = (T*)a.out + (size_t)row * a.out_row_stride + (size_t)vhead * a.hd;
    const int seq = a.token_seq[row];
    if (seq < 0) {
        for (int d = lane; d < a.hd; d += 32) o[d] = from_f32<T>(0.f);
        return;
    }
    const int pos = a.positions[row];
    const int kvh = head / (a.nqh / a.nkh);
    const int val_h = a.value_heads > 1 ? vhead - head * a.value_heads : kvh;
    const float scale = a.head_scale ? a.scale * a.head_scale[head] : a.scale;
    const T* q = (const T*)a.q + (size_t)row * a.q_row_stride + (size_t)head * a.hd;
    for (int d = lane; d < a.hd; d += 32) qs[d] = to_f32(q[d]);
    __syncwarp();

    const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    float m = -INFINITY, l = 0.f;
    float acc[ATTN_SIMPLE_MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < ATTN_SIMPLE_MAX_HD / 32; ++i) acc[i] = 0.f;
    const int* table = a.page_table + (size_t)seq * a.table_cols;
    const size_t head_stride = (size_t)a.page_size * a.hd;

    const int kept = a.keep_first < lo ? a.keep_first : lo;      // kept first positions that the window has left
    for (int part = kept > 0 ? 0 : 1; part < 2; ++part) {
    const int end = part ? pos + 1 : kept;
    for (int j0 = part ? lo : 0; j0 < end; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        const T* vrow = nullptr;
        if (j < end) {
            const int block = j / a.page_size, off = j - block * a.page_size;
            int page = (block < a.table_cols) ? table[block] : -1;
            if (page < 0 || page >= a.num_pages) {      // never followed: flag it and read page 0 instead
                atomicExch(a.error_flag, 1);
                page = 0;
            }
            const T* kbase = (const T*)a.cache + ((size_t)page * 2 * a.nkh + kvh) * head_stride + (size_t)off * a.hd;
            vrow = kbase + (size_t)(a.nkh + val_h - kvh) * head_stride;
            float dot = 0.f;
            for (int d = 0; d < a.hd; ++d) dot = fmaf(qs[d], to_f32(kbase[d]), dot);
            s = dot * scale;
        }
        const float cmax = warp_max(s);
        const float m_new = fmaxf(m, cmax);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float p = (j < end) ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
        m = m_new;
        ps[lane] = p;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < ATTN_SIMPLE_MAX_HD / 32; ++i) acc[i] *= corr;
        const int n_valid = min(32, end - j0);
        for (int jj = 0; jj < n_valid; ++jj) {
            const T* vr = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)vrow, jj);
            const float pj = ps[jj];
#pragma unroll
            for (int i = 0; i < ATTN_SIMPLE_MAX_HD / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < a.hd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
        __syncwarp();
    }
    }
    float corr_end = 1.f;
    if (a.has_sink) {                                // the sink joins as one more score, with no value
        const float sink = a.head_sinks ? a.head_sinks[head] : a.sink_score;
        const float m_new = fmaxf(m, sink);
        corr_end = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr_end + expf(sink - m_new);
    }
    float inv = corr_end * a.out_scale / l;
    if (a.head_gate) inv *= 1.f / (1.f + expf(-to_f32(((const T*)a.head_gate)[(size_t)row * a.gate_stride + head])));
#pragma unroll
    for (int i = 0; i < ATTN_SIMPLE_MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < a.hd) o[d] = from_f32<T>(acc[i] * inv);
    }
}

extern "C" int braid_attn_simple(const void* q, void* out, int dtype, const void* cache,
                                 const int* page_table, const int* positions, const int* token_seq,
                                 int q_row_stride, int out_row_stride, int rows, int nqh, int nkh, int hd,
                                 int page_size, int table_cols, int num_pages, int window, float scale,
                                 int has_sink, float sink_score, float out_scale, const float* head_sinks,
                                 const void* head_gate, long long gate_stride, int keep_first, const float* head_scale,
                                 int value_heads, int* error_flag, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (!error_flag) BRAID_REFUSE("attn_simple: error_flag is required");
    if (num_pages <= 0 || table_cols <= 0 || page_size <= 0) BRAID_REFUSE("attn_simple: the cache has no pages (pages=%d, table columns=%d, page size=%d)", num_pages, table_cols, page_size);
    if (nqh <= 0 || nkh <= 0 || nqh % nkh != 0) BRAID_REFUSE("attn_simple: %d query heads do not divide into %d kv heads", nqh, nkh);
    if (hd <= 0 || hd > ATTN_SIMPLE_MAX_HD) BRAID_REFUSE("attn_simple: head_dim=%d outside (0, %d]", hd, ATTN_SIMPLE_MAX_HD);
    if (value_heads != 1 && value_heads != nkh) BRAID_REFUSE("attn_simple: a head reads the values of its own kv head or of all %d, not of %d", nkh, value_heads);
    if (value_heads > 1 && head_gate) BRAID_REFUSE("attn_simple: a gate a head does not go with values of every kv head");
    if (keep_first < 0) BRAID_REFUSE("attn_simple: keep_first=%d must not be negative", keep_first);
    if (window <= 0) keep_first = 0;
    AttnSimpleArgs a{q, out, cache, page_table, positions, token_seq, q_row_stride, out_row_stride,
                     rows, nqh, nkh, hd, page_size, table_cols, num_pages, window, scale, has_sink || head_sinks != nullptr, sink_score, out_scale, error_flag, head_sinks, head_gate, gate_stride,
                     keep_first, head_scale, value_heads};
    const long long items = (long long)rows * nqh * value_heads;
    const long long blocks = (items + ATTN_SIMPLE_WARPS - 1) / ATTN_SIMPLE_WARPS;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("attn_simple: %lld (token, head) pairs exceed one launch", items);
    const size_t smem = (size_t)ATTN_SIMPLE_WARPS * (hd + 32) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32) braid_launch(attn_simple_kernel<float>, dim3((int)blocks), dim3(ATTN_SIMPLE_WARPS * 32), smem, s, a);
    else if (dtype == BRAID_BF16) braid_launch(attn_simple_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(ATTN_SIMPLE_WARPS * 32), smem, s, a);
    else BRAID_REFUSE("attn_simple: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}
