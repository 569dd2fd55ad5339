// Histogram build in the reference's own arithmetic ("fp32 mode").
//
// The reference keeps ONE float (g,h) accumulator per bin of a node in global memory and adds every stored value
// to it with atomicAdd (src/thundergbm/builder/hist_tree_builder_single.cu:203-216 for the root, :485-505 for the
// smaller child of a pair).  A bin's sum is therefore a sequential float accumulation of its values in some order,
// and when many equal values meet in one bin (first boosting round of a classification objective: every row of a
// class carries the same hessian) that accumulation drifts by a few 1e-5 relative, whatever the order.  Sums that
// are first collected per CTA and then combined -- or exact integer sums -- do not reproduce the drift, and the
// gains computed from them sit a few 1e-4 away from the reference's.  So this mode keeps the reference's scheme:
// one accumulator per (node, bin) for the whole GPU, every (row, feature) pair issues one vector reduction
// `red.global.add.v2.f32` that the L2 performs in arrival order.
//
// The L2 spreads addresses over its slices in chunks much larger than a cell, so the 57 KB of a single node's cells
// keep only a few slices busy (measured: 86 G reductions/s into 8-byte cells of one node, 163 G/s with the cells
// 64 bytes apart, 181 G/s into the compact cells of 64 nodes).  Levels with few histograms therefore write their
// cells `cell_stride` float2 apart; the evaluation kernels read them with the same stride.
//
// The fixed-point kernels (k_hist, k_hist_sparse) remain the deterministic mode.
#pragma once
#include "tgbm_kernels.cuh"

namespace tgbm {

__device__ __forceinline__ void red_add_gh(float2 *cell, float g, float h) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(cell), "f"(g), "f"(h) : "memory");
}

constexpr int F32_THREADS = 512;
// First global bin of up to 256 features, passed to the dense kernel BY VALUE: kernel parameters live in the constant
// bank, so the unrolled feature loop reads them without touching the load/store pipe the reductions already saturate
// (with the offsets in shared memory the top stall was the memory-instruction queue).
struct CutOffsets { int v[256]; };

// Dense layout.  grid = (CTAs, feature groups of 32); a CTA takes half a 1024-record tile of the level's tile
// sequence at a time, a thread one record: its 32 bin bytes, its gradient pair, one reduction per present feature.
template <bool GATHER>
static __global__ void __launch_bounds__(F32_THREADS)
k_hist_f32(const unsigned char *__restrict__ bins, int Fpad, int F, const int *__restrict__ rec_idx,
           const float2 *__restrict__ rec_gh, const int4 *__restrict__ seq, const TreeCtl *__restrict__ ctl,
           const int *__restrict__ cut_ptr, float2 *__restrict__ slab, int B, int cell_stride,
           const __grid_constant__ CutOffsets cuts, int cuts_in_param) {
    __shared__ int s_cut[32];
    const int f0 = blockIdx.y * 32, nf = min(32, F - f0);
    if (!cuts_in_param) {  // more than 256 features: the offsets of the CTA's group through shared memory
        if (threadIdx.x < 32) s_cut[threadIdx.x] = threadIdx.x < nf ? cut_ptr[f0 + threadIdx.x] : 0;
        __syncthreads();
    }
    constexpr int PER_TILE = HIST_THREADS / F32_THREADS;
    const int units = ctl->n_hist_tiles * PER_TILE;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int4 e = seq[u / PER_TILE];  // first record, records, histogram slot
        const int q = (u % PER_TILE) * F32_THREADS + threadIdx.x;
        if (q >= e.y) continue;
        const int p = e.x + q;
        const int r = GATHER ? rec_idx[p] : p;
        const float2 v = rec_gh[p];
        const uint4 *row = reinterpret_cast<const uint4 *>(bins + (size_t)r * Fpad + f0);
        const uint4 a = row[0], b = row[1];
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        float2 *dst = slab + (size_t)e.z * B * cell_stride;
#pragma unroll
        for (int f = 0; f < 32; ++f) {
            const uint32_t bin = (w[f >> 2] >> (8 * (f & 3))) & 0xffu;
            if (f < nf && bin != MISSING_BIN) {
                const int first_bin = cuts_in_param ? cuts.v[(f0 + f) & 255] : s_cut[f];
                red_add_gh(dst + (size_t)(first_bin + bin) * cell_stride, v.x, v.y);
            }
        }
    }
}

// CSR layout: a warp per record, lanes over the row's stored values (global bin ids).
template <bool GATHER>
static __global__ void __launch_bounds__(F32_THREADS)
k_hist_sparse_f32(const int *__restrict__ row_ptr, const int *__restrict__ bin, const int *__restrict__ rec_idx,
                  const float2 *__restrict__ rec_gh, const HistWork *__restrict__ work, const int *__restrict__ tile_base,
                  const TreeCtl *__restrict__ ctl, float2 *__restrict__ slab, int B, int cell_stride) {
    const int total = ctl->n_hist_tiles, nwork = ctl->n_hist_work;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int W = F32_THREADS / 32;
    for (int t = blockIdx.x; t < total; t += gridDim.x) {
        int lo = 0, hi = nwork - 1;  // the work item of tile t: last w with tile_base[w] <= t
        while (lo < hi) {
            const int mid = (lo + hi + 1) / 2;
            if (tile_base[mid] <= t) lo = mid; else hi = mid - 1;
        }
        const HistWork it = work[lo];
        float2 *dst = slab + (size_t)it.slab * B * cell_stride;
        const int first = (t - tile_base[lo]) * HIST_THREADS, last = min(it.count, first + HIST_THREADS);
        for (int q = first + warp; q < last; q += W) {
            const int p = it.begin + q;
            const int r = GATHER ? rec_idx[p] : p;
            const float2 v = rec_gh[p];
            const int j1 = row_ptr[r + 1];
            for (int j = row_ptr[r] + lane; j < j1; j += 32) red_add_gh(dst + (size_t)bin[j] * cell_stride, v.x, v.y);
        }
    }
}

// Root sums of the round's gradients per class (Tree::init2, src/thundergbm/tree.cu:31, a thrust::reduce over float
// pairs in the reference): fp64 partial sums per block in a fixed order, then one warp per class.
constexpr int SUM_BLOCKS = 256;
static __global__ void __launch_bounds__(256)
k_sum_gh(const float2 *__restrict__ gh, int n, double *__restrict__ partial) {
    __shared__ double wg[8], wh[8];
    const int k = blockIdx.y;
    double sg = 0, sh = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float2 v = gh[(size_t)k * n + i];
        sg += (double)v.x; sh += (double)v.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { sg += __shfl_xor_sync(0xffffffffu, sg, o); sh += __shfl_xor_sync(0xffffffffu, sh, o); }
    if ((threadIdx.x & 31) == 0) { wg[threadIdx.x >> 5] = sg; wh[threadIdx.x >> 5] = sh; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double tg = 0, th = 0;
        for (int w = 0; w < 8; ++w) { tg += wg[w]; th += wh[w]; }
        partial[((size_t)k * gridDim.x + blockIdx.x) * 2] = tg;
        partial[((size_t)k * gridDim.x + blockIdx.x) * 2 + 1] = th;
    }
}
static __global__ void k_sum_gh_final(const double *__restrict__ partial, int nb, double *__restrict__ out) {
    const int k = blockIdx.x;
    double tg = 0, th = 0;
    for (int i = threadIdx.x; i < nb; i += 32) { tg += partial[((size_t)k * nb + i) * 2]; th += partial[((size_t)k * nb + i) * 2 + 1]; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { tg += __shfl_xor_sync(0xffffffffu, tg, o); th += __shfl_xor_sync(0xffffffffu, th, o); }
    if (threadIdx.x == 0) { out[2 * k] = tg; out[2 * k + 1] = th; }
}

}  // namespace tgbm
