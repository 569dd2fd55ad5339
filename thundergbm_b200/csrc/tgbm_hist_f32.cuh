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
// The L2 performs the reductions that aim at one line one after the other, so cells packed 16 to a line are its
// worst case (measured with the bare reductions of 10.5 M rows x 28: 87 G/s into 8-byte cells of one node, 165 G/s
// with the cells 64 bytes apart, 176 G/s at 128 bytes, 190 G/s at 256 bytes, 165 G/s at 512 bytes; the same order with
// 8 or 64 nodes).  The histograms are therefore built with their cells `cell_stride` float2 apart (32 = 256 bytes
// wherever the spread buffer has room); the evaluation kernels read them with the same stride.
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

// ---- bulk-copy staging of the record tiles (gather levels) ---------------------------------------------------------
// At the levels below the root a CTA reads, for every unit of F32_THREADS records, the unit's row ids and gradient
// pairs: two contiguous pieces of rec_idx / rec_gh.  They are brought into shared memory by the copy engine
// (cp.async.bulk global -> shared, completion counted on an mbarrier; a plain one-CTA copy from this GPU's own memory)
// one unit ahead of the threads, so that the only global loads left on a thread's critical path are its bin row and the
// reductions.  A bulk copy needs 16-byte aligned addresses and sizes: a unit starts at any record, so the copy starts
// at the aligned record before it and is a few records longer; the threads index from the remainder.
// Every wait on the barrier is bounded; a wait that runs out records itself in ctl->error and the CTA stops.
constexpr int STAGE_IDX = F32_THREADS + 4;   // ints per staged row-id piece   (2064 bytes)
constexpr int STAGE_GH = F32_THREADS + 2;    // float2 per staged gradient piece (4112 bytes)
constexpr int STAGE_WAIT_LIMIT = 1 << 22;

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
// true when the phase with the given parity has completed; false after STAGE_WAIT_LIMIT polls
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    for (int it = 0; it < STAGE_WAIT_LIMIT; ++it) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

// Dense layout.  grid = (CTAs, feature groups of 32); a CTA takes half a 1024-record tile of the level's tile
// sequence at a time, a thread one record: its 32 bin bytes, its gradient pair, one reduction per present feature.
template <bool GATHER>
static __global__ void __launch_bounds__(F32_THREADS)
k_hist_f32(const unsigned char *__restrict__ bins, int Fpad, int F, const int *__restrict__ rec_idx,
           const float2 *__restrict__ rec_gh, const int4 *__restrict__ seq, TreeCtl *__restrict__ ctl,
           const int *__restrict__ cut_ptr, float2 *__restrict__ slab, int B, int cell_stride,
           const __grid_constant__ CutOffsets cuts, int cuts_in_param, int staged) {
    __shared__ int s_cut[32];
    __shared__ __align__(16) int s_idx[2][STAGE_IDX];
    __shared__ __align__(16) float2 s_gh[2][STAGE_GH];
    __shared__ __align__(8) uint64_t s_bar[2];
    __shared__ int s_fail;
    const int f0 = blockIdx.y * 32, nf = min(32, F - f0);
    if (!cuts_in_param) {  // more than 256 features: the offsets of the CTA's group through shared memory
        if (threadIdx.x < 32) s_cut[threadIdx.x] = threadIdx.x < nf ? cut_ptr[f0 + threadIdx.x] : 0;
    }
    constexpr int PER_TILE = HIST_THREADS / F32_THREADS;
    const int units = ctl->n_hist_tiles * PER_TILE;
    const bool stage = GATHER && staged;
    auto unit_first = [&](int u) { const int4 e = seq[u / PER_TILE]; return e.x + (u % PER_TILE) * F32_THREADS; };
    auto issue = [&](int u, int buf) {  // thread 0: both pieces of unit u into buffer buf
        const int p0 = unit_first(u);
        const int a_idx = p0 & ~3, a_gh = p0 & ~1;
        mbar_expect_tx(&s_bar[buf], (uint32_t)(STAGE_IDX * sizeof(int) + STAGE_GH * sizeof(float2)));
        bulk_g2s(s_idx[buf], rec_idx + a_idx, (uint32_t)(STAGE_IDX * sizeof(int)), &s_bar[buf]);
        bulk_g2s(s_gh[buf], rec_gh + a_gh, (uint32_t)(STAGE_GH * sizeof(float2)), &s_bar[buf]);
    };
    if (stage) {
        if (threadIdx.x == 0) {
            mbar_init(&s_bar[0], 1); mbar_init(&s_bar[1], 1);
            s_fail = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    __syncthreads();
    // A CTA takes a contiguous run of the unit sequence, so that at any moment the CTAs of the grid work on different
    // nodes: with all of them on the same node (units dealt out round-robin) every reduction in flight aims at that one
    // node's 57 KB of cells, the regime the L2 handles worst (86 G reductions/s against 181 G/s over 64 nodes).
    const int run = (units + (int)gridDim.x - 1) / (int)gridDim.x;
    const int u_begin = min((int)blockIdx.x * run, units), u_end = min(u_begin + run, units);
    if (stage && threadIdx.x == 0 && u_begin < u_end) issue(u_begin, 0);
    int n_done = 0;  // units this CTA has consumed: buffer = n_done & 1, parity = (n_done >> 1) & 1
    for (int u = u_begin; u < u_end; ++u, ++n_done) {
        const int4 e = seq[u / PER_TILE];  // first record, records, histogram slot
        const int q = (u % PER_TILE) * F32_THREADS + threadIdx.x;
        int r = -1;
        float2 v = make_float2(0.f, 0.f);
        if (stage) {
            const int buf = n_done & 1;
            if (threadIdx.x == 0 && u + 1 < u_end) issue(u + 1, buf ^ 1);  // one unit ahead
            if (!mbar_wait(&s_bar[buf], (n_done >> 1) & 1)) { s_fail = 1; atomicCAS(&ctl->error, 0, 0x40000000 | u); }
            const int p0 = e.x + (u % PER_TILE) * F32_THREADS;
            if (q < e.y) { r = s_idx[buf][(p0 & 3) + threadIdx.x]; v = s_gh[buf][(p0 & 1) + threadIdx.x]; }
            __syncthreads();  // every thread holds its record: the buffer may be refilled two units from now
            if (s_fail) {  // leave only when the copy that is still on its way has landed (bounded as well)
                if (threadIdx.x == 0 && u + 1 < u_end) mbar_wait(&s_bar[buf ^ 1], ((n_done + 1) >> 1) & 1);
                return;
            }
            if (threadIdx.x == 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        } else if (q < e.y) {
            const int p = e.x + q;
            r = GATHER ? rec_idx[p] : p;
            v = rec_gh[p];
        }
        if (r < 0) continue;
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
// spread cells (`stride` float2 apart) -> consecutive cells: what the ranks all-reduce
static __global__ void k_compact_cells(const float2 *__restrict__ spread, float2 *__restrict__ compact, size_t cells, int stride) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < cells; i += (size_t)gridDim.x * blockDim.x)
        compact[i] = spread[i * (size_t)stride];
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
