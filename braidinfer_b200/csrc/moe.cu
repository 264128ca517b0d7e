// Mixture of experts: routing, the plan that sorts a step's (token, choice) pairs by expert, the
// experts' matrix products over those sorted rows, and the weighted sum back into the residual stream.
//
// Routing (one warp a token): s = softmax(z) over all experts; the experts form `groups` equal groups of
// neighbours, a group's score is its largest s, and only experts of the `keep` best groups can be chosen;
// the `top` allowed experts with the largest s are chosen (ties: the lower index); their weights are
// their s divided by the sum of the chosen s (+ 1e-20), times `mult` (a constant factor the caller wants
// on the layer's output).  Everything float32.  `sigmoid` routing instead scores every expert by itself,
// s = 1 / (1 + exp(-z)), chooses the same way, and leaves the chosen scores as the weights (times `mult`), not
// renormalised.
//
// The plan: every chosen (token, choice) pair gets a slot in an array ordered by expert, each expert's run
// padded to a multiple of `tile` slots, so that a tile of slots belongs to one expert and the products can
// run tile by tile with the sizes known only on the device.  Which slot of its expert's run a pair gets
// does not touch any number: every output row is a sum over k in a fixed order whatever its slot.
// Launch sizes depend on the step's shape alone (an upper bound of tiles), so a CUDA graph can replay them.
#include "common.cuh"
#include "mma_tile.cuh"

// ------------------------------------------------------------------ routing
struct MoeRouteArgs {
    const float* logits;      // [rows, experts]
    int* idx;                 // [rows, top]
    float* wgt;               // [rows, top]
    int rows, experts, top, groups, keep;
    float mult;
    int sigmoid;              // scores are sigmoids of the logits and the weights are the chosen scores as they are
};

#define MOE_ROUTE_WARPS 4

__global__ void __launch_bounds__(MOE_ROUTE_WARPS * 32)
moe_route_kernel(MoeRouteArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];          // per warp: [experts] scores, [groups] group scores
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * MOE_ROUTE_WARPS + warp;
    if (row >= a.rows) return;
    float* s = smem + (size_t)warp * (a.experts + a.groups);
    float* gs = s + a.experts;
    const float* z = a.logits + (size_t)row * a.experts;
    if (a.sigmoid) {
        for (int e = lane; e < a.experts; e += 32) s[e] = 1.f / (1.f + expf(-z[e]));
    } else {
        float mx = -INFINITY;
        for (int e = lane; e < a.experts; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < a.experts; e += 32) {
            const float p = expf(z[e] - mx);
            s[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        const float inv = 1.f / sum;
        for (int e = lane; e < a.experts; e += 32) s[e] *= inv;
    }
    __syncwarp();
    const int per = a.experts / a.groups;
    for (int g = lane; g < a.groups; g += 32) {
        float m = -INFINITY;
        for (int i = 0; i < per; ++i) m = fmaxf(m, s[g * per + i]);
        gs[g] = m;
    }
    __syncwarp();
    // the `keep` best groups stay; the others are closed by marking their score negative
    // (a kept group's score is made > 2, a softmax score never is)
    for (int k = 0; k < a.keep; ++k) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int g = lane; g < a.groups; g += 32) {
            const float v = gs[g];
            if (v <= 2.f && (v > best || (v == best && g < bi))) { best = v; bi = g; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (lane == 0 && bi != 0x7fffffff) gs[bi] = 3.f;
        __syncwarp();
    }
    // the `top` largest scores among experts of kept groups; a chosen expert's score is then hidden
    float chosen_sum = 0.f;
    for (int k = 0; k < a.top; ++k) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < a.experts; e += 32) {
            const float v = s[e];
            if (v >= 0.f && gs[e / per] > 2.f && (v > best || (v == best && e < bi))) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (bi == 0x7fffffff) { bi = -1; best = 0.f; }      // fewer allowed experts than `top`
        if (lane == 0) {
            a.idx[(size_t)row * a.top + k] = bi;
            a.wgt[(size_t)row * a.top + k] = best;
            if (bi >= 0) s[bi] = -1.f;
        }
        chosen_sum += best;
        __syncwarp();
    }
    const float norm = a.sigmoid ? a.mult : a.mult / (chosen_sum + 1e-20f);
    __syncwarp();
    for (int k = lane; k < a.top; k += 32) a.wgt[(size_t)row * a.top + k] *= norm;
}

extern "C" int braid_moe_route(const float* logits, int* idx, float* wgt, int rows, int experts, int top,
                               int groups, int keep, float mult, int sigmoid, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (experts <= 0 || top <= 0 || top > experts) BRAID_REFUSE("moe_route: top=%d of %d experts", top, experts);
    if (groups <= 0 || experts % groups || keep <= 0 || keep > groups) BRAID_REFUSE("moe_route: %d experts in %d groups, %d kept", experts, groups, keep);
    const size_t smem = (size_t)MOE_ROUTE_WARPS * (experts + groups) * sizeof(float);
    if (smem > 48 * 1024) BRAID_REFUSE("moe_route: %d experts are more than one block's shared memory holds", experts);
    MoeRouteArgs a{logits, idx, wgt, rows, experts, top, groups, keep, mult, sigmoid};
    braid_launch(moe_route_kernel, dim3((rows + MOE_ROUTE_WARPS - 1) / MOE_ROUTE_WARPS), dim3(MOE_ROUTE_WARPS * 32), smem,
                 (cudaStream_t)stream, a);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ the plan
// One block.  idx [rows * top] holds each pair's expert (-1: none); pairs of padding rows (token_seq < 0)
// take no slot.  Outputs: slot_pair [cap] (pair of each slot, -1 for padding slots), pair_slot [rows * top]
// (slot of each pair, -1 for none), tile_expert [max_tiles], meta[0] = tiles in use.
#define MOE_MAX_EXPERTS 1024

__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ idx, const int* __restrict__ token_seq, int* __restrict__ slot_pair,
                int* __restrict__ pair_slot, int* __restrict__ tile_expert, int* __restrict__ meta,
                int rows, int top, int experts, int tile, int max_tiles) {
    pdl_trigger();
    pdl_wait();
    __shared__ int count[MOE_MAX_EXPERTS];
    __shared__ int start[MOE_MAX_EXPERTS];
    const int pairs = rows * top;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    for (int i = threadIdx.x; i < max_tiles * tile; i += blockDim.x) slot_pair[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = (token_seq[i / top] >= 0) ? idx[i] : -1;
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < experts; ++e) {
            start[e] = run;
            run += (count[e] + tile - 1) / tile;
        }
        meta[0] = run < max_tiles ? run : max_tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        const int n = (count[e] + tile - 1) / tile;
        for (int t = 0; t < n; ++t)
            if (start[e] + t < max_tiles) tile_expert[start[e] + t] = e;
        count[e] = 0;                       // from here on: the cursor within the expert's run
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = (token_seq[i / top] >= 0) ? idx[i] : -1;
        int slot = -1;
        if (e >= 0 && e < experts) {
            slot = start[e] * tile + atomicAdd(&count[e], 1);
            if (slot < max_tiles * tile) slot_pair[slot] = i; else slot = -1;
        }
        pair_slot[i] = slot;
    }
}

extern "C" int braid_moe_plan(const int* idx, const int* token_seq, int* slot_pair, int* pair_slot, int* tile_expert,
                              int* meta, int rows, int top, int experts, int tile, int max_tiles, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (experts <= 0 || experts > MOE_MAX_EXPERTS) BRAID_REFUSE("moe_plan: %d experts (at most %d)", experts, MOE_MAX_EXPERTS);
    if (tile <= 0 || tile % 16) BRAID_REFUSE("moe_plan: the tile of %d slots must be a multiple of 16", tile);
    braid_launch(moe_plan_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, idx, token_seq, slot_pair, pair_slot,
                 tile_expert, meta, rows, top, experts, tile, max_tiles);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ the experts' products, plain
// Units of 16 slots x 64 outputs; 256 threads, each one slot and four outputs; float32 FMA in a fixed
// order along k.  MODE 0: act[slot, j] = silu(x[token] . gate_e[j]) * (x[token] . up_e[j]), the input rows
// gathered through slot_pair.  MODE 1: y[slot, j] = act[slot] . down_e[j].  MODE 2 (experts without a gate):
// act[slot, j] = relu(x[token] . up_e[j])^2, the input rows gathered like MODE 0's, w0 the up matrices.
// With `in_wgt` (MODE 0) a pair's weight multiplies the expert's input instead of its output: the expert sees w x, and
// since its first products are linear, gate and up are multiplied by w in float32 before the activation,
// act = silu(w (x . gate)) * (w (x . up)); the weighted sum then adds the pairs with weight 1.
struct MoeGemmArgs {
    const void* x;            // MODE 0: [rows, ldx] the layer's normed input; MODE 1: act [slots, ldx]
    const void* w0;           // MODE 0: gate [experts, J, K]; MODE 1: down [experts, J, K]
    const void* w1;           // MODE 0: up [experts, J, K]
    void* out;                // [slots, ldo]
    const int* slot_pair;
    const int* tile_expert;
    const int* meta;
    long long ldx, ldo;
    int J, K, top, tile;
    const float* in_wgt;      // MODE 0: [rows * top] a weight a pair on the expert's input; or null
};

template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_gemm_simt_kernel(MoeGemmArgs a) {
    pdl_trigger();
    pdl_wait();
    __shared__ float xs[16][16 + 1];        // [k][slot]
    __shared__ float w0s[16][64 + 4];       // [k][output]
    __shared__ float w1s[MODE == 0 ? 16 : 1][64 + 4];
    const int unit = blockIdx.y;                             // 16 slots
    const int t = unit * 16 / a.tile;
    if (t >= a.meta[0]) return;
    const int e = a.tile_expert[t];
    const int slot0 = unit * 16;
    const int m0 = blockIdx.x * 64;
    const int ts = threadIdx.x >> 4, tj = threadIdx.x & 15;  // ts: slot, tj: group of four outputs
    const int my_pair = a.slot_pair[slot0 + ts];
    // the row this thread fetches for the x tile: thread (r = tid >> 4, c = tid & 15) loads x[slot r][k0 + c]
    const long long src_row = (MODE != 1) ? (my_pair >= 0 ? my_pair / a.top : -1) : (slot0 + ts);
    const T* w0 = (const T*)a.w0 + (size_t)e * a.J * a.K;
    const T* w1 = (MODE == 0) ? (const T*)a.w1 + (size_t)e * a.J * a.K : nullptr;
    float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < a.K; k0 += 16) {
        {
            const int k = k0 + tj;
            xs[tj][ts] = (src_row >= 0 && k < a.K) ? to_f32(((const T*)a.x)[(size_t)src_row * a.ldx + k]) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int el = threadIdx.x + i * 256;            // 0..1023: 64 outputs x 16 k
            const int r = el >> 4, c = el & 15;
            const int k = k0 + c, m = m0 + r;
            const bool ok = (m < a.J && k < a.K);
            w0s[c][r] = ok ? to_f32(w0[(size_t)m * a.K + k]) : 0.f;
            if (MODE == 0) w1s[c][r] = ok ? to_f32(w1[(size_t)m * a.K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            const float xv = xs[kk][ts];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc0[j] = fmaf(xv, w0s[kk][tj * 4 + j], acc0[j]);
                if (MODE == 0) acc1[j] = fmaf(xv, w1s[kk][tj * 4 + j], acc1[j]);
            }
        }
        __syncthreads();
    }
    T* o = (T*)a.out + (size_t)(slot0 + ts) * a.ldo;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int m = m0 + tj * 4 + j;
        if (m >= a.J) continue;
        if (MODE == 0) {
            const float wi = (a.in_wgt && my_pair >= 0) ? a.in_wgt[my_pair] : 1.f;
            const float g = acc0[j] * wi;
            o[m] = from_f32<T>(my_pair >= 0 ? g / (1.f + expf(-g)) * (acc1[j] * wi) : 0.f);
        } else if (MODE == 2) {
            const float r = fmaxf(acc0[j], 0.f);
            o[m] = from_f32<T>(my_pair >= 0 ? r * r : 0.f);
        } else {
            o[m] = from_f32<T>(acc0[j]);
        }
    }
}

extern "C" int braid_moe_gemm_simt(const void* x, const void* w0, const void* w1, void* out, const int* slot_pair,
                                   const int* tile_expert, const int* meta, int dtype, int mode, long long ldx,
                                   long long ldo, int J, int K, int top, int tile, int max_tiles, const float* in_wgt,
                                   void* stream) {
    if (max_tiles <= 0 || J <= 0) return BRAID_OK;
    if (K <= 0) BRAID_REFUSE("moe_gemm: k=%d must be positive", K);
    if (tile <= 0 || tile % 16) BRAID_REFUSE("moe_gemm: the tile of %d slots must be a multiple of 16", tile);
    if (in_wgt && mode != 0) BRAID_REFUSE("moe_gemm: a weight on the expert's input goes with the gated first product (mode 0)");
    MoeGemmArgs a{x, w0, w1, out, slot_pair, tile_expert, meta, ldx, ldo, J, K, top, tile, in_wgt};
    const long long units = (long long)max_tiles * (tile / 16);
    if (units > 65535) BRAID_REFUSE("moe_gemm: %lld units of 16 slots exceed the grid limit", units);
    dim3 grid((J + 63) / 64, (unsigned)units);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32 && mode == 0) braid_launch(moe_gemm_simt_kernel<float, 0>, grid, dim3(256), 0, s, a);
    else if (dtype == BRAID_F32 && mode == 1) braid_launch(moe_gemm_simt_kernel<float, 1>, grid, dim3(256), 0, s, a);
    else if (dtype == BRAID_BF16 && mode == 0) braid_launch(moe_gemm_simt_kernel<__nv_bfloat16, 0>, grid, dim3(256), 0, s, a);
    else if (dtype == BRAID_BF16 && mode == 1) braid_launch(moe_gemm_simt_kernel<__nv_bfloat16, 1>, grid, dim3(256), 0, s, a);
    else if (dtype == BRAID_F32 && mode == 2) braid_launch(moe_gemm_simt_kernel<float, 2>, grid, dim3(256), 0, s, a);
    else if (dtype == BRAID_BF16 && mode == 2) braid_launch(moe_gemm_simt_kernel<__nv_bfloat16, 2>, grid, dim3(256), 0, s, a);
    else BRAID_REFUSE("moe_gemm: unknown dtype %d or mode %d", dtype, mode);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ the experts' products on the tensor cores
// bfloat16, mma.sync with float32 accumulators (mma_tile.cuh).  One CTA a plan tile of BM slots (the plan's
// tile is BM) and BN outputs.  MODE 0 multiplies the gathered rows with the expert's gate and up matrices at
// once and stores silu(gate) * up; MODE 1 multiplies the activations with the down matrix; MODE 2 multiplies the
// gathered rows with the expert's up matrix alone and stores relu(.)^2.
template <int BM, int BN, int MODE>
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(MoeGemmArgs a) {
    constexpr int NB = MODE == 0 ? 2 : 1;
    using Tile = MmaTile<BM, BN, (BM >= 64 ? 2 : 1), (BM >= 64 ? 2 : 4), NB>;
    extern __shared__ __align__(16) unsigned char moe_smem[];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    if (t >= a.meta[0]) return;
    const int e = a.tile_expert[t];
    const int slot0 = t * BM, m0 = blockIdx.x * BN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int ACH = BM * 4 / 128 > 0 ? BM * 4 / 128 : 1;
    constexpr int BCH = BN * 4 / 128;
    const __nv_bfloat16* a_rows[ACH];
    const __nv_bfloat16* b_rows[NB][BCH];
    const __nv_bfloat16* x = (const __nv_bfloat16*)a.x;
#pragma unroll
    for (int i = 0; i < ACH; ++i) {
        const int r = (tid + i * 128) >> 2;
        a_rows[i] = nullptr;
        if (r < BM) {
            if (MODE != 1) {
                const int pair = a.slot_pair[slot0 + r];
                if (pair >= 0) a_rows[i] = x + (size_t)(pair / a.top) * a.ldx;
            } else {
                a_rows[i] = x + (size_t)(slot0 + r) * a.ldx;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < BCH; ++i) {
        const int m = m0 + ((tid + i * 128) >> 2);
        b_rows[0][i] = m < a.J ? (const __nv_bfloat16*)a.w0 + ((size_t)e * a.J + m) * a.K : nullptr;
        if (MODE == 0) b_rows[NB - 1][i] = m < a.J ? (const __nv_bfloat16*)a.w1 + ((size_t)e * a.J + m) * a.K : nullptr;
    }
    float acc[NB][Tile::MI][Tile::NI][4];
    Tile::run(acc, (__nv_bfloat16*)moe_smem, a_rows, b_rows, a.K, a.w0);
    const int wm0 = (warp / (BM >= 64 ? 2 : 4)) * (BM / (BM >= 64 ? 2 : 1)), wn0 = (warp % (BM >= 64 ? 2 : 4)) * (BN / (BM >= 64 ? 2 : 4));
    __nv_bfloat16* out = (__nv_bfloat16*)a.out;
    const bool pairs_ok = (a.ldo & 1) == 0;
#pragma unroll
    for (int mi = 0; mi < Tile::MI; ++mi)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int slot = slot0 + wm0 + mi * 16 + (lane >> 2) + half * 8;
            const int pair_here = MODE == 1 ? 0 : a.slot_pair[slot];
            const bool live = pair_here >= 0;
            const float wi = (MODE == 0 && a.in_wgt && live) ? a.in_wgt[pair_here] : 1.f;
#pragma unroll
            for (int ni = 0; ni < Tile::NI; ++ni) {
                const int col = m0 + wn0 + ni * 8 + 2 * (lane & 3);
                float v0, v1;
                if (MODE == 0) {
                    const float g0 = acc[0][mi][ni][half * 2] * wi, g1 = acc[0][mi][ni][half * 2 + 1] * wi;
                    v0 = live ? g0 / (1.f + expf(-g0)) * (acc[NB - 1][mi][ni][half * 2] * wi) : 0.f;
                    v1 = live ? g1 / (1.f + expf(-g1)) * (acc[NB - 1][mi][ni][half * 2 + 1] * wi) : 0.f;
                } else if (MODE == 2) {
                    const float r0 = fmaxf(acc[0][mi][ni][half * 2], 0.f), r1 = fmaxf(acc[0][mi][ni][half * 2 + 1], 0.f);
                    v0 = live ? r0 * r0 : 0.f;
                    v1 = live ? r1 * r1 : 0.f;
                } else {
                    v0 = acc[0][mi][ni][half * 2];
                    v1 = acc[0][mi][ni][half * 2 + 1];
                }
                __nv_bfloat16* o = out + (size_t)slot * a.ldo + col;
                if (pairs_ok && col + 1 < a.J) *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(v0, v1);
                else {
                    if (col < a.J) o[0] = __float2bfloat16_rn(v0);
                    if (col + 1 < a.J) o[1] = __float2bfloat16_rn(v1);
                }
            }
        }
}

extern "C" int braid_moe_gemm_mma(const void* x, const void* w0, const void* w1, void* out, const int* slot_pair,
                                  const int* tile_expert, const int* meta, int mode, long long ldx, long long ldo,
                                  int J, int K, int top, int tile, int max_tiles, const float* in_wgt, void* stream) {
    if (max_tiles <= 0 || J <= 0) return BRAID_OK;
    if (K <= 0 || K % 8 || ldx % 8) BRAID_REFUSE("moe_gemm_mma: k=%d and the row stride %lld must be multiples of 8", K, ldx);
    if (((uintptr_t)x | (uintptr_t)w0 | (uintptr_t)w1) & 15) BRAID_REFUSE("moe_gemm_mma: operands must start on 16 bytes");
    if (tile != 16 && tile != 64) BRAID_REFUSE("moe_gemm_mma: the plan's tile must be 16 or 64 slots, not %d", tile);
    if (max_tiles > 65535) BRAID_REFUSE("moe_gemm_mma: %d tiles exceed the grid limit", max_tiles);
    if (in_wgt && mode != 0) BRAID_REFUSE("moe_gemm: a weight on the expert's input goes with the gated first product (mode 0)");
    MoeGemmArgs a{x, w0, w1, out, slot_pair, tile_expert, meta, ldx, ldo, J, K, top, tile, in_wgt};
    cudaStream_t s = (cudaStream_t)stream;
    // the down product over tiles of 64 slots takes 128 outputs a CTA (its rows are fetched half as often: 0.36 -> 0.29 ms
    // at 2,048 tokens of width 2048); gate+up with its two accumulators stays at 64 (at 128 it needs 237 registers and
    // was 8 % slower), and so do tiles of 16
#define MOE_MMA(BM, BN, MODE)                                                                                   \
    do {                                                                                                        \
        using T_ = MmaTile<BM, BN, (BM >= 64 ? 2 : 1), (BM >= 64 ? 2 : 4), (MODE == 0 ? 2 : 1)>;                \
        static bool attr_set = false;                                                                           \
        if (!attr_set && T_::SMEM_BYTES > 48 * 1024) {                                                          \
            cudaError_t e_ = cudaFuncSetAttribute(moe_gemm_mma_kernel<BM, BN, MODE>,                            \
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, T_::SMEM_BYTES); \
            if (e_ != cudaSuccess) BRAID_REFUSE("moe_gemm_mma: shared memory: %s", cudaGetErrorString(e_));      \
            attr_set = true;                                                                                    \
        }                                                                                                       \
        braid_launch(moe_gemm_mma_kernel<BM, BN, MODE>, dim3((J + BN - 1) / BN, (unsigned)max_tiles), dim3(128), \
                     (size_t)T_::SMEM_BYTES, s, a);                                                             \
    } while (0)
    if (tile == 64 && mode == 0) MOE_MMA(64, 64, 0);
    else if (tile == 64 && mode == 1) MOE_MMA(64, 128, 1);
    else if (tile == 16 && mode == 0) MOE_MMA(16, 64, 0);
    else if (tile == 16 && mode == 1) MOE_MMA(16, 64, 1);
    else if (tile == 64 && mode == 2) MOE_MMA(64, 128, 2);
    else if (tile == 16 && mode == 2) MOE_MMA(16, 64, 2);
    else BRAID_REFUSE("moe_gemm_mma: unknown mode %d", mode);
#undef MOE_MMA
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ the weighted sum
// h[row, :] += sum over the row's choices k, in the order of k, of wgt[row, k] * y[pair_slot[row, k], :]
// (wgt null: every weight is 1, for experts whose weight went into their input).
template <typename T>
__global__ void moe_combine_kernel(float* __restrict__ h, const T* __restrict__ y, const int* __restrict__ pair_slot,
                                   const float* __restrict__ wgt, int rows, int width, int top, long long ldy) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int slot = pair_slot[(size_t)row * top + k];
            if (slot >= 0) acc = fmaf(wgt ? wgt[(size_t)row * top + k] : 1.f, to_f32(y[(size_t)slot * ldy + c]), acc);
        }
        h[(size_t)row * width + c] += acc;
    }
}

extern "C" int braid_moe_combine(float* h, const void* y, int y_dtype, const int* pair_slot, const float* wgt,
                                 int rows, int width, int top, long long ldy, void* stream) {
    if (rows <= 0) return BRAID_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : 128;
    if (y_dtype == BRAID_F32) braid_launch(moe_combine_kernel<float>, dim3(rows), dim3(threads), 0, s, h, (const float*)y, pair_slot, wgt, rows, width, top, ldy);
    else if (y_dtype == BRAID_BF16) braid_launch(moe_combine_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, s, h, (const __nv_bfloat16*)y, pair_slot, wgt, rows, width, top, ldy);
    else BRAID_REFUSE("moe_combine: unknown dtype code %d", y_dtype);
    BRAID_LAUNCH_CHECK();
}
