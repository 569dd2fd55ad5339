// LambdaRank gradients and ranking metrics on the GPU, one CTA per query group.
// The reference computes both on the host with OpenMP (src/thundergbm/objective/ranking_obj.cpp:21-91,
// src/thundergbm/metric/rank_metric.cpp) and copies scores and gradients across PCIe every round.
// Its partner sampling is seeded from std::rand() inside a parallel loop and is not reproducible, so
// only the distribution is kept: every document draws one uniform partner outside its label bucket,
// here from a counter-based hash of (seed, round, global group id, position).
#pragma once
#include <algorithm>
#include <cmath>
#include <vector>

#include "tgbm_comm.h"
#include "tgbm_device.cuh"

namespace tgbm {

constexpr int RANK_MAX_GROUP = 4096;

__device__ inline uint32_t desc_key(float v) {  // larger float -> smaller key
    uint32_t u = __float_as_uint(v);
    if (u == 0x80000000u) u = 0;  // -0.0f == 0.0f
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ~u;
}

// sort `n` (key, idx) pairs ascending by (key, idx); arrays hold P >= n slots, P a power of two
__device__ inline void block_bitonic(unsigned long long *key, int *idx, int n, int P) {
    for (int i = threadIdx.x; i < P; i += blockDim.x)
        if (i >= n) { key[i] = ~0ull; idx[i] = 0x7fffffff; }
    __syncthreads();
    for (int k = 2; k <= P; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < P; i += blockDim.x) {
                const int l = i ^ j;
                if (l > i) {
                    const bool up = (i & k) == 0;
                    const unsigned long long a = key[i], b = key[l];
                    const int ia = idx[i], ib = idx[l];
                    const bool gt = a > b || (a == b && ia > ib);
                    if (gt == up) { key[i] = b; key[l] = a; idx[i] = ib; idx[l] = ia; }
                }
            }
            __syncthreads();
        }
    }
}

__device__ inline float disc_gain(int label, int rank, const float *__restrict__ log2tab) {
    // NDCG::discounted_gain, include/thundergbm/metric/ranking_metric.h:41-43; log2tab[r] = log2f(r + 2)
    return __fdiv_rn((float)((1 << label) - 1), log2tab[rank]);
}

// LambdaRank::get_gradient for one query group per CTA
static __global__ void __launch_bounds__(256)
k_lambdarank(const int *__restrict__ gptr, const float *__restrict__ y, const float *__restrict__ yp, const float *__restrict__ idcg,
             const float *__restrict__ log2tab, int ndcg, uint32_t seed, const RoundState *__restrict__ rs, uint32_t group_offset,
             float2 *__restrict__ gh, unsigned *__restrict__ maxbits) {
    extern __shared__ __align__(16) unsigned char sm[];
    const uint32_t round = (uint32_t)rs->round;  // read on the device: the launch is the same every round
    const int k = blockIdx.x;
    const int s0 = gptr[k], len = gptr[k + 1] - s0;
    int P = 1;
    while (P < len) P <<= 1;
    unsigned long long *key = reinterpret_cast<unsigned long long *>(sm);
    int *idx = reinterpret_cast<int *>(key + P);
    float *lab = reinterpret_cast<float *>(idx + P);   // label at sorted position
    float *sc = lab + P;                               // score at sorted position
    int *hi = reinterpret_cast<int *>(sc + P);         // per position l: sorted position of the higher document
    int *lo = hi + P;
    float *lam = reinterpret_cast<float *>(lo + P);
    float *hes = lam + P;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        key[i] = ((unsigned long long)desc_key(y[s0 + i]) << 32) | desc_key(yp[s0 + i]);
        idx[i] = i;
    }
    __syncthreads();
    block_bitonic(key, idx, len, P);
    for (int i = threadIdx.x; i < len; i += blockDim.x) { lab[i] = y[s0 + idx[i]]; sc[i] = yp[s0 + idx[i]]; }
    __syncthreads();
    const float id = ndcg ? idcg[k] : 1.f;
    for (int l = threadIdx.x; l < len; l += blockDim.x) {
        // label bucket [i, j) of position l (labels descend)
        const float L = lab[l];
        int a = 0, b = l;
        while (a < b) { const int m = (a + b) / 2; if (lab[m] == L) b = m; else a = m + 1; }
        const int i = a;
        a = l; b = len;
        while (a < b) { const int m = (a + b) / 2; if (lab[m] == L) a = m + 1; else b = m; }
        const int j = a;
        const int nleft = i, nright = len - j;
        hi[l] = -1; lo[l] = -1; lam[l] = 0.f; hes[l] = 0.f;
        if (nleft + nright != 0) {
            const uint32_t r = mix32(seed, round, group_offset + (uint32_t)k, (uint32_t)l);
            const int m = (int)(((uint64_t)r * (uint32_t)(nleft + nright)) >> 32);
            int high, low;
            if (m < nleft) { high = m; low = l; } else { high = l; low = m + j - i; }
            float dz = 1.f;
            if (ndcg) {
                if (id == 0.f) dz = 0.f;
                else {
                    const float a1 = disc_gain((int)lab[high], high, log2tab), b1 = disc_gain((int)lab[low], low, log2tab);
                    const float a2 = disc_gain((int)lab[high], low, log2tab), b2 = disc_gain((int)lab[low], high, log2tab);
                    dz = __fdiv_rn(__fsub_rn(__fsub_rn(__fadd_rn(a1, b1), a2), b2), id);
                }
            }
            const float adz = fabsf(dz);
            const float rho = __fdiv_rn(1.0f, __fadd_rn(1.0f, portable_expf(__fsub_rn(sc[high], sc[low]))));
            hi[l] = high; lo[l] = low;
            lam[l] = -__fmul_rn(adz, rho);
            hes[l] = __fmul_rn(2.0f, fmaxf(__fmul_rn(__fmul_rn(adz, rho), __fsub_rn(1.0f, rho)), 1e-16f));
        }
    }
    __syncthreads();
    // every document sums what it receives in ascending l, the order of the reference's sequential loop
    float mg = 0.f, mh = 0.f;
    for (int t = threadIdx.x; t < len; t += blockDim.x) {
        float g = 0.f, h = 0.f;
        for (int l = 0; l < len; ++l) {
            if (hi[l] == t) { g = __fadd_rn(g, lam[l]); h = __fadd_rn(h, hes[l]); }
            else if (lo[l] == t) { g = __fadd_rn(g, -lam[l]); h = __fadd_rn(h, hes[l]); }
        }
        gh[s0 + idx[t]] = make_float2(g, h);
        mg = fmaxf(mg, fabsf(g)); mh = fmaxf(mh, h);
    }
    unsigned ua = __float_as_uint(mg), ub = __float_as_uint(mh);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { ua = max(ua, __shfl_xor_sync(0xffffffffu, ua, o)); ub = max(ub, __shfl_xor_sync(0xffffffffu, ub, o)); }
    if ((threadIdx.x & 31) == 0) { atomicMax(maxbits, ua); atomicMax(maxbits + 1, ub); }
}

// NDCG / MAP of one query group per CTA (src/thundergbm/metric/rank_metric.cpp:42-100):
// documents ordered by score descending (ties by row), sequential sums in rank order
static __global__ void __launch_bounds__(256)
k_rank_metric(const int *__restrict__ gptr, const float *__restrict__ y, const float *__restrict__ yp, const float *__restrict__ idcg,
              const float *__restrict__ log2tab, int ndcg, float *__restrict__ group_score) {
    extern __shared__ __align__(16) unsigned char sm[];
    const int k = blockIdx.x;
    const int s0 = gptr[k], len = gptr[k + 1] - s0;
    int P = 1;
    while (P < len) P <<= 1;
    unsigned long long *key = reinterpret_cast<unsigned long long *>(sm);
    int *idx = reinterpret_cast<int *>(key + P);
    if (ndcg && idcg[k] == 0.f) { if (threadIdx.x == 0) group_score[k] = 1.f; return; }
    for (int i = threadIdx.x; i < len; i += blockDim.x) { key[i] = desc_key(yp[s0 + i]); idx[i] = i; }
    __syncthreads();
    block_bitonic(key, idx, len, P);
    if (threadIdx.x == 0) {
        if (ndcg) {
            float dcg = 0.f;
            for (int i = 0; i < len; ++i) dcg = __fadd_rn(dcg, disc_gain((int)y[s0 + idx[i]], i, log2tab));
            group_score[k] = __fdiv_rn(dcg, idcg[k]);
        } else {
            int nh = 0;
            double ap = 0;
            for (int i = 0; i < len; ++i)
                if (y[s0 + idx[i]] != 0.f) { nh++; ap += (double)nh / (i + 1); }
            group_score[k] = nh ? (float)(ap / nh) : 1.f;
        }
    }
}

static __global__ void k_rank_metric_sum(const float *__restrict__ group_score, int n_group, double *__restrict__ out) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        double s = 0;
        for (int i = 0; i < n_group; ++i) s += (double)group_score[i];
        *out = s;
    }
}
static __global__ void k_rank_metric_final(const double *__restrict__ sum, long long n_group_total, float *__restrict__ out) {
    if (threadIdx.x == 0 && blockIdx.x == 0) *out = (float)(*sum / (double)n_group_total);
}

struct RankState {
    int n_group = 0, max_len = 0, N = 0;
    long long n_group_total = 0;
    uint32_t group_offset = 0;  // global index of this rank's first group
    DevBuf<int> gptr;
    DevBuf<float> idcg, log2tab, y, group_score;
    DevBuf<double> sum;

    // Rank-local checks of the query groups.  Called before the first collective of Booster::init, so that a rank with
    // bad groups stops together with its peers instead of leaving them inside a collective.
    static void validate(const DataSet &ds, int n_rows) {
        long long total = 0;
        int longest = 0;
        for (int g : ds.group) { TGBM_CHECK(g >= 0, "negative query group size"); total += g; longest = std::max(longest, g); }
        TGBM_CHECK(total == n_rows, "group sizes must add up to the number of rows");
        TGBM_CHECK(longest <= RANK_MAX_GROUP, "query groups of more than 4096 rows are not supported");
    }

    // first_group / total_groups: global index of this rank's first query group and the number of groups over all ranks
    // (the partner sampling is keyed by the global group index, the metric is the mean over all groups)
    void init(const DataSet &ds, int objective, int n_rows, cudaStream_t stream, long long first_group, long long total_groups) {
        N = n_rows;
        const float *labels = ds.yv ? ds.yv : ds.y.data();
        n_group = (int)ds.group.size();
        std::vector<int> h(n_group + 1, 0);
        for (int i = 0; i < n_group; ++i) { h[i + 1] = h[i] + ds.group[i]; max_len = std::max(max_len, ds.group[i]); }
        validate(ds, n_rows);
        // NDCG::get_IDCG (rank_metric.cpp:102-123), host code in the reference as well
        std::vector<float> hid(std::max(n_group, 1), 0.f);
        std::vector<float> ltab(std::max(max_len, 1));
        for (int r = 0; r < (int)ltab.size(); ++r) ltab[r] = log2f((float)(r + 1 + 1));
        if (objective == RANK_NDCG)
            for (int k = 0; k < n_group; ++k) {
                std::vector<float> s(labels + h[k], labels + h[k + 1]);
                std::sort(s.begin(), s.end(), std::greater<float>());
                float v = 0.f;
                for (size_t i = 0; i < s.size(); ++i) v += (float)((1 << (int)s[i]) - 1) / ltab[i];
                hid[k] = v;
            }
        gptr.alloc(n_group + 1); idcg.alloc(hid.size()); log2tab.alloc(ltab.size()); y.alloc(std::max(n_rows, 1));
        group_score.alloc(std::max(n_group, 1)); sum.alloc(1);
        TGBM_CUDA(cudaMemcpyAsync(gptr.p, h.data(), sizeof(int) * h.size(), cudaMemcpyHostToDevice, stream));
        TGBM_CUDA(cudaMemcpyAsync(idcg.p, hid.data(), sizeof(float) * hid.size(), cudaMemcpyHostToDevice, stream));
        TGBM_CUDA(cudaMemcpyAsync(log2tab.p, ltab.data(), sizeof(float) * ltab.size(), cudaMemcpyHostToDevice, stream));
        TGBM_CUDA(cudaMemcpyAsync(y.p, labels, sizeof(float) * n_rows, cudaMemcpyHostToDevice, stream));
        TGBM_CUDA(cudaStreamSynchronize(stream));
        n_group_total = total_groups;
        group_offset = (uint32_t)first_group;
        idcg_used = objective == RANK_NDCG;
        int P = 1;
        while (P < max_len) P <<= 1;
        const int smem = 40 * P;
        if (smem > 48 * 1024) {
            TGBM_CUDA(cudaFuncSetAttribute(k_lambdarank, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        }
    }
    int pow2_len() const { int P = 1; while (P < max_len) P <<= 1; return P; }

    void gradient(const RoundState *rs, uint32_t seed, const float *yp, float2 *gh, unsigned *maxbits, cudaStream_t stream) {
        if (!n_group) return;
        TGBM_CUDA(cudaMemsetAsync(gh, 0, sizeof(float2) * (size_t)N, stream));
        const int P = pow2_len();
        k_lambdarank<<<n_group, 256, 40 * (size_t)P, stream>>>(gptr.p, y.p, yp, idcg.p, log2tab.p, idcg_used, seed, rs,
                                                             group_offset, gh, maxbits);
    }
    // `out` null: the sum of the group scores stays in `sum` (the caller finishes the metric)
    void metric(int objective, const float *yp, float *out, const Comm *comm, long long, cudaStream_t stream) {
        const int P = pow2_len();
        if (n_group) k_rank_metric<<<n_group, 256, 12 * (size_t)P, stream>>>(gptr.p, y.p, yp, idcg.p, log2tab.p, objective == RANK_NDCG, group_score.p);
        k_rank_metric_sum<<<1, 32, 0, stream>>>(group_score.p, n_group, sum.p);
        if (comm && comm->active()) comm->allreduce(sum.p, 1, Comm::F64, Comm::SUM, stream);
        if (out) k_rank_metric_final<<<1, 32, 0, stream>>>(sum.p, n_group_total, out);
    }
    int idcg_used = 0;
};

}  // namespace tgbm
