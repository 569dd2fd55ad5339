// CPU restatement of ThunderGBM's 1-GPU histogram tree-building path
// (HistTreeBuilder_single and everything it calls).
//
// THIS IS TEST INFRASTRUCTURE.  It is the checker the CUDA path is compared
// against and the timed host-core baseline.  Only tests, the smoke entry and
// the benchmark's cpu_baseline / reference arm may load it; the product never
// links, imports or falls back to it.
//
// Parity pinning: checked by tests/test_oracle_golden.py against (a) outputs of
// the reference itself (built by oracle/build_ref.sh, run on a B200 through
// oracle/ref_harness.cu; packed under tests/golden/) and (b) the known-answer
// tests of the reference's own suite (src/test/test_metrics.cpp:70,84,96,
// src/test/test_tree.cpp:68, src/test/test_dataset.cpp:178-181).
//
// Every function cites the reference file:line it restates (paths relative to
// the reference project root).
//
// Two histogram arithmetics:
//   hist_mode 0  "fp32"  : float accumulation in ascending row order, float
//                          per-feature prefix sums -- one admissible ordering of
//                          the reference's unordered float atomics.
//   hist_mode 1  "exact" : gradients rounded to a power-of-two grid
//                          (quant_bits value bits under the per-round maximum),
//                          accumulated in fp64 in ascending row order.  Every
//                          partial sum is an integer multiple of the grid below
//                          2^53, so the fixed-order fp64 reduction is exact and
//                          equals the sum in any other order bit for bit.  This
//                          is the deterministic mode of the CUDA path.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <numeric>
#include <string>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---------------------------------------------------------------- data types
// include/thundergbm/tree.h:14-42 -- 48-byte node record, also the model-file record
struct TreeNode {
    int final_id, lch_index, rch_index, parent_index;
    float gain, base_weight;
    int split_feature_id;
    float split_value;
    unsigned char split_bid;
    bool default_right, is_leaf, is_valid, is_pruned;
    unsigned char pad_[3];
    float sum_g, sum_h;
};
static_assert(sizeof(TreeNode) == 48, "TreeNode must match the reference's 48-byte record");

struct GH { float g, h; };  // include/thundergbm/common.h:43-84

enum Objective { REG_LINEAR = 0, REG_LOGISTIC = 1, BINARY_LOGISTIC = 2, MULTI_SOFTMAX = 3, MULTI_SOFTPROB = 4,
                 RANK_PAIRWISE = 5, RANK_NDCG = 6 };

}  // namespace

extern "C" {
struct TgoParam {
    int depth, n_trees, max_num_bin, objective, num_class;
    float lambda, gamma, min_child_weight, rt_eps, learning_rate;
    int hist_mode;    // 0 fp32 row-order, 1 exact (quantised fp64)
    int quant_bits;   // value bits of the grid in hist_mode 1
    int n_threads;    // OpenMP threads (0 = all)
    int keep_nid;     // keep ins2node_id of every tree (tests only)
    int portable_exp; // 1: use the portable expf shared with the CUDA path, 0: libm expf
    unsigned rank_seed;
    int bagging;                // RowSampler::do_bagging
    float column_sampling_rate; // Shard::column_sampling, 1 = off
    unsigned sample_seed;
    int multi_shards;  // 0: HistTreeBuilder_single; D >= 1: HistTreeBuilder with the columns split over D devices
    int exact_builder; // 1: ExactTreeBuilder (tree_method = exact): every distinct value of a node is a candidate
};
}

namespace {

// ------------------------------------------------------------- portable expf
// Cody-Waite range reduction + degree-5 polynomial (the classic single-precision
// scheme); built only from IEEE fp32 mul/fma/rint so that the CPU and the GPU
// produce identical bits.  Replaces CUDA's expf (include/thundergbm/objective/
// regression_obj.h:144-154, src/thundergbm/objective/multiclass_obj.cu:22-28).
inline float pow2i(int e) {  // 2^e for e in [-126,127]
    uint32_t u = (uint32_t)(e + 127) << 23;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
inline float portable_expf(float x) {
    if (!(x <= 88.72283f)) return x != x ? x : INFINITY;
    if (x < -103.9f) return 0.0f;
    float n = rintf(x * 1.44269504088896341f);
    float r = fmaf(n, -0.693359375f, x);
    r = fmaf(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    float e = fmaf(p, r * r, r) + 1.0f;
    int k = (int)n;
    int k1 = k / 2, k2 = k - k1;
    return (e * pow2i(k1)) * pow2i(k2);
}

struct Ctx {
    TgoParam p;
    int N = 0, F = 0, K = 1;  // rows, features, trees per round
    std::vector<int> row_ptr, col;
    std::vector<float> val, y;
    std::vector<float> label;  // distinct labels (classification)
    std::vector<int> gptr;     // query-group offsets
    // cuts
    std::vector<float> cut_val;
    std::vector<int> cut_ptr, cut_fid;
    std::vector<int> bin;  // global bin id per stored value
    // model
    float base_score = 0;
    int n_nodes = 0;
    std::vector<TreeNode> trees;  // [round][k][n_nodes]
    std::vector<float> metric;    // per round
    std::vector<float> ypred;     // [K][N]
    std::vector<int> nid_keep;    // [tree][N]
    std::vector<float> idcg;
    std::vector<float> hist_dump;  // level histograms of the first tree (tests): see tgo_first_tree_hist
    std::vector<double> quant_scale;  // per round: 2^s_g, 2^s_h
    std::vector<double> round_seconds;
    std::vector<float> gain2;  // [tree][n_nodes]: runner-up |gain| at every evaluated node (how decisive the split was)
    std::vector<unsigned char> ignored;  // column-sampling mask of the running round (empty = no sampling)
    // exact builder: the stored values by column, largest first (SparseColumns::csr2csc_gpu, sparse_columns.cu:20-93,127)
    std::vector<int64_t> csc_ptr;
    std::vector<int> csc_row;
    std::vector<float> csc_val;
    double train_seconds = 0, init_seconds = 0;
    float expf_(float x) const { return p.portable_exp ? portable_expf(x) : expf(x); }
};

double now_s() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// ---------------------------------------------------------------- data set
// src/thundergbm/dataset.cpp:83-101 group_label(): labels are cast to int, sorted, uniqued;
// y becomes the index of its (float) value in that list, 0 when it is not in the list.
void group_label(Ctx &c) {
    std::vector<int> t(c.y.begin(), c.y.end());
    std::sort(t.begin(), t.end());
    t.erase(std::unique(t.begin(), t.end()), t.end());
    std::map<float, int> m;
    c.label.clear();
    for (int v : t) { m[(float)v] = (int)c.label.size(); c.label.push_back((float)v); }
    for (auto &v : c.y) { auto it = m.find(v); v = it == m.end() ? 0.f : (float)it->second; }
}

// src/thundergbm/hist_cut.cu:205-286 get_cut_points_single + unique_by_flag2:
// per feature the ascending distinct stored values; with u distinct values and s = u / max_bin
// (integer division) keep all when s == 0, else the values at positions 0, s, 2s, ..., (max_bin-1)s.
void find_cuts(Ctx &c) {
    const int F = c.F, mb = c.p.max_num_bin;
    std::vector<int64_t> cnt(F + 1, 0);
    const int64_t nnz = c.row_ptr[c.N];
    for (int64_t i = 0; i < nnz; ++i) cnt[c.col[i] + 1]++;
    for (int f = 0; f < F; ++f) cnt[f + 1] += cnt[f];
    std::vector<float> byc(nnz);
    {
        std::vector<int64_t> pos(cnt.begin(), cnt.end() - 1);
        for (int64_t i = 0; i < nnz; ++i) byc[pos[c.col[i]]++] = c.val[i];
    }
    std::vector<std::vector<float>> per(F);
#pragma omp parallel for schedule(dynamic, 1)
    for (int f = 0; f < F; ++f) {
        float *b = byc.data() + cnt[f], *e = byc.data() + cnt[f + 1];
        std::sort(b, e);
        e = std::unique(b, e);  // operator== : -0.0f and 0.0f merge like thrust::unique
        const int u = (int)(e - b);
        const int s = u / mb;
        auto &o = per[f];
        if (s == 0) o.assign(b, e);
        else { o.resize(mb); for (int j = 0; j < mb; ++j) o[j] = b[(int64_t)s * j]; }
    }
    c.cut_ptr.assign(F + 1, 0);
    for (int f = 0; f < F; ++f) c.cut_ptr[f + 1] = c.cut_ptr[f] + (int)per[f].size();
    c.cut_val.resize(c.cut_ptr[F]);
    c.cut_fid.resize(c.cut_ptr[F]);
    for (int f = 0; f < F; ++f)
        for (size_t j = 0; j < per[f].size(); ++j) {
            c.cut_val[c.cut_ptr[f] + j] = per[f][j] == 0.0f ? 0.0f : per[f][j];  // canonical +0
            c.cut_fid[c.cut_ptr[f] + j] = f;
        }
}

// src/thundergbm/builder/hist_tree_builder_single.cu:81-119 get_bin_ids: upper bound over
// [begin, end-1] => bin = min(#cuts <= v, n_cuts-1), stored as global id.
void bin_ids(Ctx &c) {
    const int64_t nnz = c.row_ptr[c.N];
    c.bin.resize(nnz);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nnz; ++i) {
        const int f = c.col[i];
        int lo = c.cut_ptr[f], hi = c.cut_ptr[f + 1] - 1;
        const float v = c.val[i];
        while (lo < hi) {
            const int mid = lo + (hi - lo) / 2;
            if (c.cut_val[mid] <= v) lo = mid + 1; else hi = mid;
        }
        c.bin[i] = lo;
    }
}

// ------------------------------------------------- column-sharded builder (n_device > 1)
// src/thundergbm/sparse_columns.cu:95-102 csr2csc_gpu: device d owns the columns [d*(F/D), (d+1)*(F/D)), the
// last device also the remainder.
inline void shard_columns(int F, int D, int d, int &first, int &count) {
    const int ave = F / D;
    first = d * ave;
    count = d < D - 1 ? ave : F - first;
}

// src/thundergbm/hist_cut.cu:104-187 get_cut_points3 + unique_by_flag, once per device on its own columns:
// every stored value v of local column j becomes t = v + j*(m+1) with m the largest value on the device, all t
// are sorted descending, the column ids are laid over them by COUNT (largest id first), runs of equal t collapse
// to their first entry, t goes back to t - j*(m+1) and a stable sort by column id groups the result.  The round
// trip is done in float (each direction one fused multiply-add, checked against the reference's own cut points), so for j > 0 the candidates are the stored values rounded to the spacing of floats near
// j*(m+1), and columns whose values reach below -1 trade candidates with their neighbours; both effects are part of
// what the reference computes and are kept.  From the n candidates of a column every (n / max_bin)-th is kept
// (all when n < max_bin), at most max_bin, in descending order.
void find_cuts_multi(Ctx &c) {
    const int F = c.F, mb = c.p.max_num_bin, D = c.p.multi_shards;
    const int64_t nnz = c.row_ptr[c.N];
    std::vector<int64_t> cnt(F + 1, 0);
    for (int64_t i = 0; i < nnz; ++i) cnt[c.col[i] + 1]++;
    for (int f = 0; f < F; ++f) cnt[f + 1] += cnt[f];
    std::vector<float> byc(nnz);
    {
        std::vector<int64_t> pos(cnt.begin(), cnt.end() - 1);
        for (int64_t i = 0; i < nnz; ++i) byc[pos[c.col[i]]++] = c.val[i];
    }
    std::vector<std::vector<float>> per(F);
    for (int d = 0; d < D; ++d) {
        int first, ncol;
        shard_columns(F, D, d, first, ncol);
        const int64_t lo = cnt[first], hi = cnt[first + ncol], n = hi - lo;
        if (n == 0) continue;
        float m = byc[lo];
        for (int64_t i = lo; i < hi; ++i) m = std::max(m, byc[i]);
        const float step = m + 1;
        std::vector<float> t(n);
        for (int j = 0; j < ncol; ++j)
            for (int64_t i = cnt[first + j]; i < cnt[first + j + 1]; ++i) {
                const float v = byc[i];
                t[i - lo] = fmaf((float)j, step, v);  // nvcc contracts the functor's `v + j * step` into one fma
            }
        std::sort(t.begin(), t.end(), std::greater<float>());
        std::vector<int> flag(n);
        {
            int64_t o = 0;
            for (int j = ncol - 1; j >= 0; --j)
                for (int64_t i = cnt[first + j]; i < cnt[first + j + 1]; ++i) flag[o++] = j;
        }
        std::vector<std::vector<float>> cand(ncol);
        for (int64_t i = 0; i < n; ++i) {
            if (i > 0 && t[i] == t[i - 1]) continue;  // thrust::unique_by_key keeps the first of a run
            const int j = flag[i];
            cand[j].push_back(fmaf(-(float)j, step, t[i]));
        }
        for (int j = 0; j < ncol; ++j) {
            const auto &a = cand[j];
            const int u = (int)a.size(), s = u / mb;
            auto &o = per[first + j];
            if (s == 0) o = a;
            else { o.resize(mb); for (int k = 0; k < mb; ++k) o[k] = a[(int64_t)s * k]; }
        }
    }
    c.cut_ptr.assign(F + 1, 0);
    for (int f = 0; f < F; ++f) c.cut_ptr[f + 1] = c.cut_ptr[f] + (int)per[f].size();
    c.cut_val.resize(c.cut_ptr[F]);
    c.cut_fid.resize(c.cut_ptr[F]);
    for (int f = 0; f < F; ++f)
        for (size_t j = 0; j < per[f].size(); ++j) {
            c.cut_val[c.cut_ptr[f] + j] = per[f][j];
            c.cut_fid[c.cut_ptr[f] + j] = f;
        }
}

// src/thundergbm/builder/hist_tree_builder.cu:15-64 get_bin_ids: over the column's cut points as stored (meant to
// descend) the search of :31-42 -- first position whose cut is <= v, the last position when there is none.
void bin_ids_multi(Ctx &c) {
    const int64_t nnz = c.row_ptr[c.N];
    c.bin.resize(nnz);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nnz; ++i) {
        const int f = c.col[i];
        int left = c.cut_ptr[f], right = c.cut_ptr[f + 1] - 1;
        const float v = c.val[i];
        while (left != right) {
            const int mid = left + (right - left) / 2;
            if (c.cut_val[mid] <= v) right = mid; else left = mid + 1;
        }
        c.bin[i] = left;
    }
}

// src/thundergbm/sparse_columns.cu:20-93 csr2csc_gpu + :127 the per-column sort by value, descending and stable
// (rows of equal value stay in ascending order)
void build_csc(Ctx &c) {
    const int F = c.F;
    const int64_t nnz = c.row_ptr[c.N];
    c.csc_ptr.assign(F + 1, 0);
    for (int64_t i = 0; i < nnz; ++i) c.csc_ptr[c.col[i] + 1]++;
    for (int f = 0; f < F; ++f) c.csc_ptr[f + 1] += c.csc_ptr[f];
    c.csc_row.resize(nnz); c.csc_val.resize(nnz);
    std::vector<int64_t> pos(c.csc_ptr.begin(), c.csc_ptr.end() - 1);
    for (int r = 0; r < c.N; ++r)
        for (int j = c.row_ptr[r]; j < c.row_ptr[r + 1]; ++j) {
            const int64_t o = pos[c.col[j]]++;
            c.csc_row[o] = r; c.csc_val[o] = c.val[j];
        }
#pragma omp parallel for schedule(dynamic, 1)
    for (int f = 0; f < F; ++f) {
        const int64_t a = c.csc_ptr[f], b = c.csc_ptr[f + 1];
        std::vector<int64_t> idx(b - a);
        for (int64_t i = 0; i < b - a; ++i) idx[i] = a + i;
        std::stable_sort(idx.begin(), idx.end(), [&](int64_t x, int64_t y) { return c.csc_val[x] > c.csc_val[y]; });
        std::vector<int> rr(b - a); std::vector<float> vv(b - a);
        for (int64_t i = 0; i < b - a; ++i) { rr[i] = c.csc_row[idx[i]]; vv[i] = c.csc_val[idx[i]]; }
        std::copy(rr.begin(), rr.end(), c.csc_row.begin() + a);
        std::copy(vv.begin(), vv.end(), c.csc_val.begin() + a);
    }
}

// ---------------------------------------------------------------- objectives
inline float sigmoidf_(const Ctx &c, float x) { return 1 / (1 + c.expf_(-x)); }

// include/thundergbm/metric/ranking_metric.h:41-43
inline float discounted_gain(int label, int rank) { return ((1 << label) - 1) / log2f(rank + 1 + 1); }

// src/thundergbm/metric/rank_metric.cpp:102-123 NDCG::get_IDCG
void compute_idcg(Ctx &c) {
    const int G = (int)c.gptr.size() - 1;
    c.idcg.assign(G, 0.f);
    for (int k = 0; k < G; ++k) {
        std::vector<float> s(c.y.begin() + c.gptr[k], c.y.begin() + c.gptr[k + 1]);
        std::sort(s.begin(), s.end(), std::greater<float>());
        for (size_t i = 0; i < s.size(); ++i) c.idcg[k] += discounted_gain((int)s[i], (int)i);
    }
}

// counter-based generator shared with the CUDA path: the reference seeds std::mt19937 from
// std::rand() inside an OpenMP loop (src/thundergbm/objective/ranking_obj.cpp:53), which is not
// reproducible run to run, so only its distribution (one uniform partner outside the label
// bucket) is restated.
inline uint32_t mix32(uint32_t a, uint32_t b, uint32_t c3, uint32_t d) {
    uint64_t z = ((uint64_t)a << 32 | b) * 0x9E3779B97F4A7C15ull + ((uint64_t)c3 << 32 | d);
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (uint32_t)(z >> 32);
}

// src/thundergbm/objective/ranking_obj.cpp:21-91 LambdaRank::get_gradient and :105-113 get_delta_z.
// Orderings made total: score descending with ties by row, then label descending, stable.
void lambdarank_gradient(const Ctx &c, int round, const float *yp, GH *gh, bool ndcg) {
    const int G = (int)c.gptr.size() - 1;
    for (int i = 0; i < c.N; ++i) gh[i] = GH{0, 0};
#pragma omp parallel for schedule(dynamic, 16)
    for (int k = 0; k < G; ++k) {
        const int s0 = c.gptr[k], len = c.gptr[k + 1] - s0;
        const float *score = yp + s0, *lab = c.y.data() + s0;
        GH *g = gh + s0;
        std::vector<int> idx(len);
        std::iota(idx.begin(), idx.end(), 0);
        std::stable_sort(idx.begin(), idx.end(), [=](int a, int b) { return score[a] > score[b]; });
        std::stable_sort(idx.begin(), idx.end(), [=](int a, int b) { return lab[a] > lab[b]; });
        for (int i = 0; i < len;) {
            int j = i + 1;
            while (j < len && lab[idx[i]] == lab[idx[j]]) j++;
            const int nleft = i, nright = len - j;
            if (nleft + nright != 0) {
                for (int l = i; l < j; ++l) {
                    const uint32_t r = mix32(c.p.rank_seed, (uint32_t)round, (uint32_t)k, (uint32_t)l);
                    const int m = (int)(((uint64_t)r * (uint32_t)(nleft + nright)) >> 32);
                    int high, low;
                    if (m < nleft) { high = m; low = l; } else { high = l; low = m + j - i; }
                    const float hl = lab[idx[high]], ll = lab[idx[low]];
                    const int hi_i = idx[high], lo_i = idx[low];
                    float dz = 1.f;
                    if (ndcg) {
                        if (c.idcg[k] == 0) dz = 0;
                        else {
                            const float a1 = discounted_gain((int)hl, high), b1 = discounted_gain((int)ll, low);
                            const float a2 = discounted_gain((int)hl, low), b2 = discounted_gain((int)ll, high);
                            dz = (a1 + b1 - a2 - b2) / c.idcg[k];
                        }
                    }
                    const float adz = fabsf(dz);
                    const float rho = 1 / (1 + c.expf_(score[hi_i] - score[lo_i]));
                    const float lambda = -adz * rho;
                    const float hess = 2 * fmaxf(adz * rho * (1 - rho), 1e-16f);
                    g[hi_i].g += lambda;  g[hi_i].h += hess;
                    g[lo_i].g += -lambda; g[lo_i].h += hess;
                }
            }
            i = j;
        }
    }
}

// include/thundergbm/objective/regression_obj.h:15-25,67-75,129-154 and
// src/thundergbm/objective/multiclass_obj.cu:7-35 (class-major gh[k*N+i])
void get_gradient(const Ctx &c, int round, const float *yp, GH *gh) {
    const int N = c.N;
    switch (c.p.objective) {
    case REG_LINEAR:
#pragma omp parallel for schedule(static)
        for (int i = 0; i < N; ++i) gh[i] = GH{yp[i] - c.y[i], 1.f};
        break;
    case REG_LOGISTIC:
    case BINARY_LOGISTIC:
#pragma omp parallel for schedule(static)
        for (int i = 0; i < N; ++i) {
            const float p = sigmoidf_(c, yp[i]);
            gh[i] = GH{p - c.y[i], fmaxf(p * (1 - p), 1e-16f)};
        }
        break;
    case MULTI_SOFTMAX:
    case MULTI_SOFTPROB: {
        const int K = c.K;
#pragma omp parallel for schedule(static)
        for (int i = 0; i < N; ++i) {
            float mx = yp[i];
            for (int k = 1; k < K; ++k) mx = fmaxf(mx, yp[(size_t)k * N + i]);
            float sum = 0;
            for (int k = 0; k < K; ++k) sum += c.expf_(yp[(size_t)k * N + i] - mx);
            for (int k = 0; k < K; ++k) {
                const float p = c.expf_(yp[(size_t)k * N + i] - mx) / sum;
                const float g = (float)k == c.y[i] ? (p - 1) : (p - 0);
                const float h = fmaxf(2 * p * (1 - p), 1e-16f);
                gh[(size_t)k * N + i] = GH{g, h};
            }
        }
        break;
    }
    case RANK_PAIRWISE: lambdarank_gradient(c, round, yp, gh, false); break;
    case RANK_NDCG: lambdarank_gradient(c, round, yp, gh, true); break;
    }
}

// ---------------------------------------------------------------- histogram arithmetic
struct Quant { double sg = 1, sh = 1; uint32_t round = 0, k = 0; };  // scales 2^s, dither stream

// Rounding to the grid is dithered: q = floor(v * scale + u) with u in [0,1) a hash of (round, class, row).
// Plain round-to-nearest would shift every row with the same gradient the same way (all rows share one
// gradient value per class in the first round), and the shifts would add up coherently in the sums.
inline double dither(uint32_t round, uint32_t k, uint32_t row, uint32_t which) {
    return (double)mix32(0x9E3779B9u + which, round, k, row) * (1.0 / 4294967296.0);
}
inline double quantize(float v, double scale, uint32_t round, uint32_t k, uint32_t row, uint32_t which) {
    return floor((double)v * scale + dither(round, k, row, which));
}

// exponent e with |m| < 2^e
inline int exp_above(float m) { int e; frexpf(m, &e); return m == 0 ? 0 : e; }

Quant choose_quant(const Ctx &c, const GH *gh, size_t n) {
    float mg = 0, mh = 0;
#pragma omp parallel for reduction(max : mg, mh) schedule(static)
    for (size_t i = 0; i < n; ++i) { mg = fmaxf(mg, fabsf(gh[i].g)); mh = fmaxf(mh, fabsf(gh[i].h)); }
    Quant q;
    q.sg = ldexp(1.0, c.p.quant_bits - exp_above(mg));
    q.sh = ldexp(1.0, c.p.quant_bits - exp_above(mh));
    return q;
}

struct Hist {            // one node: per global bin the two sums
    std::vector<double> g, h;   // exact mode: integer-valued (units of the grid); fp32 mode: float values
    void assign(int B) { g.assign(B, 0.0); h.assign(B, 0.0); }
};

struct Builder {
    Ctx &c;
    const GH *gh;
    Quant q;
    std::vector<int> nid;          // ins2node_id
    std::vector<TreeNode> nodes;
    std::vector<std::vector<Hist>> level_hist;  // [level][node in level]
    std::vector<int> rows;         // rows ordered by node (stable), rebuilt every level
    std::vector<int> node_ptr;
    Builder(Ctx &c_, const GH *gh_, Quant q_) : c(c_), gh(gh_), q(q_) {}

    inline void qrow(int r, double &g, double &h) const {
        if (c.p.hist_mode == 1) { g = quantize(gh[r].g, q.sg, q.round, q.k, (uint32_t)r, 0); h = quantize(gh[r].h, q.sh, q.round, q.k, (uint32_t)r, 1); }
        else { g = gh[r].g; h = gh[r].h; }
    }
    inline float to_f(double v, double s) const { return c.p.hist_mode == 1 ? (float)(v / s) : (float)v; }

    // src/thundergbm/builder/hist_tree_builder_single.cu:203-216 (root) and :485-505 (node):
    // hist[bin] += (g,h) of the row for every stored value of the row
    void build_hist(Hist &H, const int *rws, int n) {
        const int B = (int)c.cut_val.size();
        H.assign(B);
        if (c.p.hist_mode == 1) {
            int T = 1;
#ifdef _OPENMP
            T = c.p.n_threads > 0 ? c.p.n_threads : omp_get_max_threads();
#endif
            if ((int64_t)n * 8 < (int64_t)B || T == 1) T = 1;
            if (T == 1) {
                for (int t = 0; t < n; ++t) {
                    const int r = rws ? rws[t] : t;
                    double g, h; qrow(r, g, h);
                    for (int j = c.row_ptr[r]; j < c.row_ptr[r + 1]; ++j) { H.g[c.bin[j]] += g; H.h[c.bin[j]] += h; }
                }
            } else {  // exact sums: any grouping gives the fixed-order result bit for bit
                std::vector<Hist> part(T);
#pragma omp parallel num_threads(T)
                {
                    const int t0 = omp_get_thread_num();
                    Hist &P = part[t0];
                    P.assign(B);
                    const int lo = (int)((int64_t)n * t0 / T), hi = (int)((int64_t)n * (t0 + 1) / T);
                    for (int t = lo; t < hi; ++t) {
                        const int r = rws ? rws[t] : t;
                        double g, h; qrow(r, g, h);
                        for (int j = c.row_ptr[r]; j < c.row_ptr[r + 1]; ++j) { P.g[c.bin[j]] += g; P.h[c.bin[j]] += h; }
                    }
                }
                for (int t = 0; t < T; ++t)
                    for (int b = 0; b < B; ++b) { H.g[b] += part[t].g[b]; H.h[b] += part[t].h[b]; }
            }
        } else {
            std::vector<float> fg(B, 0.f), fh(B, 0.f);
            for (int t = 0; t < n; ++t) {
                const int r = rws ? rws[t] : t;
                const float g = gh[r].g, h = gh[r].h;
                for (int j = c.row_ptr[r]; j < c.row_ptr[r + 1]; ++j) { fg[c.bin[j]] += g; fh[c.bin[j]] += h; }
            }
            for (int b = 0; b < B; ++b) { H.g[b] = fg[b]; H.h[b] = fh[b]; }
        }
    }

    // src/thundergbm/tree.cu:8-39 Tree::init2
    void init_tree() {
        const int d = c.p.depth, n = (1 << (d + 1)) - 1;
        nodes.assign(n, TreeNode{});
        for (int i = 0; i < n; ++i) {
            TreeNode &t = nodes[i];
            t.final_id = i; t.split_feature_id = -1; t.is_valid = false;
            t.parent_index = i == 0 ? -1 : (i - 1) / 2;
            if (i < n / 2) { t.is_leaf = false; t.lch_index = 2 * i + 1; t.rch_index = 2 * i + 2; }
            else { t.is_leaf = true; t.lch_index = -1; t.rch_index = -1; }
        }
        // root sum: thrust::reduce in the reference (unordered float tree); here fp64 (exact in exact mode)
        double sg = 0, sh = 0;
        for (int i = 0; i < c.N; ++i) { double g, h; qrow(i, g, h); sg += g; sh += h; }
        nodes[0].sum_g = to_f(sg, q.sg); nodes[0].sum_h = to_f(sh, q.sh);
        nodes[0].is_valid = true;
        nodes[0].base_weight = -nodes[0].sum_g / (nodes[0].sum_h + c.p.lambda);
    }

    std::vector<float> gain2;
    struct Split { float gain = 0, gain2 = 0, miss_g = 0, miss_h = 0, l_g = 0, l_h = 0, fval = 0; bool default_right = false;
                   int nid = -1, fea = -1; unsigned char bid = 0; };

    static inline float gainf(float pg, float ph, float lg, float lh, float rg, float rh, float mcw, float lam) {
        // hist_tree_builder_single.cu:279-286 compute_gain
        if (lh >= mcw && rh >= mcw) return (lg * lg) / (lh + lam) + (rg * rg) / (rh + lam) - (pg * pg) / (ph + lam);
        return 0;
    }

    // hist_tree_builder_single.cu:257-389 (root) / :614-755 (pairs): scan, missing, gain, argmax, SplitPoint
    Split evaluate(const Hist &H, int node_id) {
        const TreeNode &nd = nodes[node_id];
        Split sp;
        if (!nd.is_valid) return sp;  // nid stays -1
        const int B = (int)c.cut_val.size();
        const float pg = nd.sum_g, ph = nd.sum_h, mcw = c.p.min_child_weight, lam = c.p.lambda;
        float best = 0, second = 0; int besti = -1; bool have = false;
        std::vector<float> Pg(B), Ph(B);
        for (int f = 0; f < c.F; ++f) {
            const int b0 = c.cut_ptr[f], b1 = c.cut_ptr[f + 1];
            if (b0 == b1) continue;
            if (!c.ignored.empty() && c.ignored[f]) continue;  // hist_tree_builder_single.cu:304,663
            if (c.p.hist_mode == 1) {
                double ag = 0, ah = 0;
                for (int i = b0; i < b1; ++i) { ag += H.g[i]; ah += H.h[i]; Pg[i] = to_f(ag, q.sg); Ph[i] = to_f(ah, q.sh); }
            } else {
                float ag = 0, ah = 0;
                for (int i = b0; i < b1; ++i) { ag += (float)H.g[i]; ah += (float)H.h[i]; Pg[i] = ag; Ph[i] = ah; }
            }
            const float mg = pg - Pg[b1 - 1], mh = ph - Ph[b1 - 1];
            for (int i = b0; i < b1; ++i) {
                float lg = 0, lh = 0;
                if (i != b0) { lg = Pg[i - 1]; lh = Ph[i - 1]; }
                const float gr = fmaxf(0.f, gainf(pg, ph, lg, lh, pg - lg, ph - lh, mcw, lam));
                const float lg2 = lg + mg, lh2 = lh + mh;
                const float gl = fmaxf(0.f, gainf(pg, ph, lg2, lh2, pg - lg2, ph - lh2, mcw, lam));
                const float gn = gl > gr ? gl : -gr;
                // arg abs max, ties -> smaller index (:330-335)
                if (!have || fabsf(gn) > fabsf(best)) { if (have) second = fmaxf(second, fabsf(best)); best = gn; besti = i; have = true; }
                else second = fmaxf(second, fabsf(gn));
            }
        }
        sp.nid = node_id;
        if (!have) { sp.fea = -1; sp.gain = 0; return sp; }
        const int f = c.cut_fid[besti], b0 = c.cut_ptr[f];
        // recompute the winner's record (:365-389)
        sp.fea = f;
        sp.gain = fabsf(best);
        sp.gain2 = second;
        sp.bid = (unsigned char)(besti - b0);
        sp.default_right = best < 0;
        // prefix of the winning feature again (Pg/Ph hold the last computed values for all features)
        sp.miss_g = pg - Pg[c.cut_ptr[f + 1] - 1];
        sp.miss_h = ph - Ph[c.cut_ptr[f + 1] - 1];
        sp.l_g = 0; sp.l_h = 0;
        sp.fval = (float)((double)(c.cut_val[b0] - fabsf(c.cut_val[b0])) - 1e-5);
        if (besti != b0) { sp.l_g = Pg[besti - 1]; sp.l_h = Ph[besti - 1]; sp.fval = c.cut_val[besti - 1]; }
        return sp;
    }

    // Column-sharded builder, src/thundergbm/builder/hist_tree_builder.cu:299-433 on every device and
    // tree_builder.cu:112-147 split_point_all_reduce across them: inclusive prefix sums along the column's bins
    // (largest values first) are the RIGHT child, the left one is the node minus it; the node's missing values go
    // right when that gains at least as much; arg abs max with ties to the smaller index inside a device and to
    // the lower device across them, which together is the smallest global bin index.  Split::l_* carry the right
    // child's sums here (SplitPoint::rch_sum_gh).
    Split evaluate_multi(const Hist &H, int node_id) {
        const TreeNode &nd = nodes[node_id];
        Split sp;
        if (!nd.is_valid) return sp;
        const int B = (int)c.cut_val.size();
        const float pg = nd.sum_g, ph = nd.sum_h, mcw = c.p.min_child_weight, lam = c.p.lambda;
        float best = 0, second = 0; int besti = -1; bool have = false;
        std::vector<float> Pg(B), Ph(B);
        for (int f = 0; f < c.F; ++f) {
            const int b0 = c.cut_ptr[f], b1 = c.cut_ptr[f + 1];
            if (b0 == b1) continue;
            if (!c.ignored.empty() && c.ignored[f]) continue;
            if (c.p.hist_mode == 1) {
                double ag = 0, ah = 0;
                for (int i = b0; i < b1; ++i) { ag += H.g[i]; ah += H.h[i]; Pg[i] = to_f(ag, q.sg); Ph[i] = to_f(ah, q.sh); }
            } else {
                float ag = 0, ah = 0;
                for (int i = b0; i < b1; ++i) { ag += (float)H.g[i]; ah += (float)H.h[i]; Pg[i] = ag; Ph[i] = ah; }
            }
            const float mg = pg - Pg[b1 - 1], mh = ph - Ph[b1 - 1];   // :288-298
            for (int i = b0; i < b1; ++i) {
                const float rg = Pg[i], rh = Ph[i];
                const float gl = fmaxf(0.f, gainf(pg, ph, pg - rg, ph - rh, rg, rh, mcw, lam));
                const float rg2 = rg + mg, rh2 = rh + mh;
                const float gr = fmaxf(0.f, gainf(pg, ph, pg - rg2, ph - rh2, rg2, rh2, mcw, lam));
                const float gn = gl > gr ? gl : -gr;
                if (!have || fabsf(gn) > fabsf(best)) { if (have) second = fmaxf(second, fabsf(best)); best = gn; besti = i; have = true; }
                else second = fmaxf(second, fabsf(gn));
            }
        }
        sp.nid = node_id;
        if (!have) { sp.fea = -1; sp.gain = 0; return sp; }
        const int f = c.cut_fid[besti], b0 = c.cut_ptr[f];
        sp.fea = f;
        sp.gain = fabsf(best);
        sp.gain2 = second;
        sp.bid = (unsigned char)(besti - b0);
        sp.default_right = best < 0;
        sp.miss_g = pg - Pg[c.cut_ptr[f + 1] - 1];
        sp.miss_h = ph - Ph[c.cut_ptr[f + 1] - 1];
        sp.l_g = Pg[besti]; sp.l_h = Ph[besti];
        sp.fval = c.cut_val[besti];
        return sp;
    }

    // src/thundergbm/builder/tree_builder.cu:9-60 update_tree (the column-sharded builder's)
    void apply_multi(const Split &sp) {
        if (sp.nid == -1) return;
        TreeNode &nd = nodes[sp.nid];
        if (sp.gain > c.p.rt_eps) {
            nd.gain = sp.gain;
            TreeNode &l = nodes[nd.lch_index], &r = nodes[nd.rch_index];
            l.is_valid = true; r.is_valid = true;
            nd.split_feature_id = sp.fea;
            nd.split_value = sp.fval;
            nd.split_bid = sp.bid;
            r.sum_g = sp.l_g; r.sum_h = sp.l_h;
            if (sp.default_right) { r.sum_g = r.sum_g + sp.miss_g; r.sum_h = r.sum_h + sp.miss_h; nd.default_right = true; }
            l.sum_g = nd.sum_g - r.sum_g; l.sum_h = nd.sum_h - r.sum_h;
            l.base_weight = -l.sum_g / (l.sum_h + c.p.lambda);
            r.base_weight = -r.sum_g / (r.sum_h + c.p.lambda);
        } else {
            nd.is_leaf = true;
            nodes[nd.lch_index].is_valid = false;
            nodes[nd.rch_index].is_valid = false;
        }
    }

    // ExactTreeBuilder::find_split (src/thundergbm/builder/exact_tree_builder.cu:15-300) for every node of the level:
    // the stored values of a (feature, node) in descending order; runs of equal value are one candidate with the run's
    // summed (g,h) (:94-111); the inclusive prefix over the runs is the RIGHT child (:114-118); missing = node sum minus
    // the last prefix (:160-167); a candidate's split value is the midpoint to the next smaller distinct value, for
    // the smallest one `v - |largest value| - rt_eps` (:137-151); gains, default direction and ties as in the
    // column-sharded histogram builder (:186-209, :218-258: smaller index, i.e. smaller feature, then larger value).
    std::vector<Split> evaluate_exact(int level) {
        const int n_level = 1 << level, off = n_level - 1;
        std::vector<Split> sps(n_level);
        struct Best { float gain = 0, second = 0; bool have = false; int fea = -1; float fval = 0, rg = 0, rh = 0, mg = 0, mh = 0; };
        std::vector<Best> best(n_level);
        const float mcw = c.p.min_child_weight, lam = c.p.lambda;
        std::vector<std::vector<int64_t>> ent(n_level);   // entries of the running feature by node, column order kept
        for (int f = 0; f < c.F; ++f) {
            const bool left_out = !c.ignored.empty() && c.ignored[f];   // :195: its candidates stay, with gain 0
            for (auto &e : ent) e.clear();
            for (int64_t i = c.csc_ptr[f]; i < c.csc_ptr[f + 1]; ++i) {
                const int n = nid[c.csc_row[i]] - off;
                if (n >= 0 && n < n_level) ent[n].push_back(i);
            }
            for (int n = 0; n < n_level; ++n) {
                const auto &e = ent[n];
                if (e.empty()) continue;
                const TreeNode &nd = nodes[off + n];
                const float pg = nd.sum_g, ph = nd.sum_h;
                // runs of equal value and their prefix sums
                std::vector<float> rv, Pg, Ph;
                if (c.p.hist_mode == 1) {
                    double ag = 0, ah = 0;
                    for (size_t t = 0; t < e.size(); ++t) {
                        double g, h; qrow(c.csc_row[e[t]], g, h);
                        ag += g; ah += h;
                        if (t + 1 == e.size() || c.csc_val[e[t + 1]] != c.csc_val[e[t]]) { rv.push_back(c.csc_val[e[t]]); Pg.push_back(to_f(ag, q.sg)); Ph.push_back(to_f(ah, q.sh)); }
                    }
                } else {
                    // run sum first (:94-111; thrust's reduce_by_key adds a run as a tree of partial sums, which stays within
                    // an ulp or two of the rounded exact sum: restated as a double sum rounded once), then the float scan
                    // over the runs (:114-118)
                    float ag = 0, ah = 0;
                    double sg = 0, sh = 0;
                    for (size_t t = 0; t < e.size(); ++t) {
                        sg += gh[c.csc_row[e[t]]].g; sh += gh[c.csc_row[e[t]]].h;
                        if (t + 1 == e.size() || c.csc_val[e[t + 1]] != c.csc_val[e[t]]) {
                            ag += (float)sg; ah += (float)sh; sg = 0; sh = 0;
                            rv.push_back(c.csc_val[e[t]]); Pg.push_back(ag); Ph.push_back(ah);
                        }
                    }
                }
                const size_t R = rv.size();
                const float mg = pg - Pg[R - 1], mh = ph - Ph[R - 1];
                Best &b = best[n];
                for (size_t t = 0; t < R; ++t) {
                    const float rg = Pg[t], rh = Ph[t];
                    const float gl = fmaxf(0.f, gainf(pg, ph, pg - rg, ph - rh, rg, rh, mcw, lam));
                    const float rg2 = rg + mg, rh2 = rh + mh;
                    const float gr = fmaxf(0.f, gainf(pg, ph, pg - rg2, ph - rh2, rg2, rh2, mcw, lam));
                    const float gn = left_out ? 0.f : (gl > gr ? gl : -gr);
                    if (!b.have || fabsf(gn) > fabsf(b.gain)) {
                        if (b.have) b.second = fmaxf(b.second, fabsf(b.gain));
                        b.have = true; b.gain = gn; b.fea = f; b.rg = rg; b.rh = rh; b.mg = mg; b.mh = mh;
                        b.fval = t + 1 == R ? (rv[t] - fabsf(rv[0])) - c.p.rt_eps : (rv[t] + rv[t + 1]) * 0.5f;
                    } else b.second = fmaxf(b.second, fabsf(gn));
                }
            }
        }
        for (int n = 0; n < n_level; ++n) {
            if (!best[n].have) continue;   // no stored value in the node: SplitPoint::nid stays -1 (:273-275)
            Split &sp = sps[n];
            const Best &b = best[n];
            sp.nid = off + n; sp.fea = b.fea; sp.gain = fabsf(b.gain); sp.gain2 = b.second; sp.bid = 0;
            sp.default_right = b.gain < 0; sp.miss_g = b.mg; sp.miss_h = b.mh; sp.l_g = b.rg; sp.l_h = b.rh; sp.fval = b.fval;
        }
        return sps;
    }

    // ExactTreeBuilder::update_ins2node_id + ins2node_id_all_reduce (exact_tree_builder.cu:303-340, :394-409): rows that
    // store the split feature compare the value with the split value, the others follow the default direction
    bool move_rows_exact() {
        bool any = false;
        std::vector<int> next(nid);
        std::vector<unsigned char> moved(c.N, 0);
        for (int f = 0; f < c.F; ++f)
            for (int64_t i = c.csc_ptr[f]; i < c.csc_ptr[f + 1]; ++i) {
                const int r = c.csc_row[i];
                const TreeNode &nd = nodes[nid[r]];
                if (nd.is_leaf || !nd.is_valid || nd.split_feature_id != f) continue;
                any = true;
                next[r] = c.csc_val[i] < nd.split_value ? nd.lch_index : nd.rch_index;
                moved[r] = 1;
            }
        if (!any) return false;   // tree_builder.cu:174-181 leaves the level loop before the default directions are applied
        for (int r = 0; r < c.N; ++r) {
            const TreeNode &nd = nodes[nid[r]];
            if (moved[r] || nd.is_leaf || !nd.is_valid) continue;
            next[r] = nd.default_right ? nd.rch_index : nd.lch_index;
        }
        nid.swap(next);
        return any;
    }

    // src/thundergbm/builder/tree_builder.cu:147-194 with ExactTreeBuilder's find_split / update_ins2node_id
    void build_exact() {
        const int d = c.p.depth;
        nid.assign(c.N, 0);
        init_tree();
        gain2.assign(nodes.size(), 0.f);
        for (int level = 0; level < d; ++level) {
            const int n_level = 1 << level, off = n_level - 1;
            std::vector<Split> sps = evaluate_exact(level);
            for (int n = 0; n < n_level; ++n) { gain2[off + n] = sps[n].gain2; apply_multi(sps[n]); }
            if (!move_rows_exact()) break;
        }
        prune();
    }

    // hist_tree_builder_single.cu:847-902 update_tree
    void apply(const Split &sp) {
        if (c.p.multi_shards > 0) { apply_multi(sp); return; }
        if (sp.nid == -1) return;
        TreeNode &nd = nodes[sp.nid];
        if (sp.gain > c.p.rt_eps) {
            nd.gain = sp.gain;
            TreeNode &l = nodes[nd.lch_index], &r = nodes[nd.rch_index];
            l.is_valid = true; r.is_valid = true;
            nd.split_feature_id = sp.fea;
            nd.split_value = sp.fval;
            nd.split_bid = sp.bid;
            l.sum_g = sp.l_g; l.sum_h = sp.l_h;
            if (!sp.default_right) { l.sum_g = l.sum_g + sp.miss_g; l.sum_h = l.sum_h + sp.miss_h; nd.default_right = false; }
            else nd.default_right = true;
            r.sum_g = nd.sum_g - l.sum_g; r.sum_h = nd.sum_h - l.sum_h;
            l.base_weight = -l.sum_g / (l.sum_h + c.p.lambda);
            r.base_weight = -r.sum_g / (r.sum_h + c.p.lambda);
        } else {
            nd.is_leaf = true;
            nodes[nd.lch_index].is_valid = false;
            nodes[nd.rch_index].is_valid = false;
        }
    }

    // hist_tree_builder_single.cu:908-1020 update_ins2node_id
    bool move_rows() {
        bool any = false;
#pragma omp parallel for schedule(static) reduction(|| : any)
        for (int i = 0; i < c.N; ++i) {
            const TreeNode &nd = nodes[nid[i]];
            if (nd.is_leaf || !nd.is_valid) continue;
            any = true;
            const int f = nd.split_feature_id, b0 = c.cut_ptr[f], b1 = c.cut_ptr[f + 1];
            const int sb = (int)nd.split_bid + b0;
            int bid = -1;
            int lo = c.row_ptr[i], hi = c.row_ptr[i + 1];  // row bins ascend with the column ids
            while (lo < hi) {
                const int mid = lo + (hi - lo) / 2, v = c.bin[mid];
                if (v >= b0 && v < b1) { bid = v; break; }
                if (v < b0) lo = mid + 1; else hi = mid;
            }
            bool left = true;
            if (c.p.multi_shards > 0) {  // hist_tree_builder.cu:455-459: bins count down from the largest values
                if ((bid == -1 && nd.default_right) || (bid >= 0 && bid <= sb)) left = false;
            } else if ((bid == -1 && nd.default_right) || (bid >= sb && bid >= 0)) left = false;
            nid[i] = left ? nd.lch_index : nd.rch_index;
        }
        return any;
    }

    // hist_tree_builder_single.cu:397-415: rows sorted by node id (stable), node_ptr per node of the level
    void partition_rows(int level) {
        const int n_level = 1 << level, off = n_level - 1;
        node_ptr.assign(n_level + 1, 0);
        for (int i = 0; i < c.N; ++i) { const int l = nid[i] - off; if (l >= 0 && l < n_level) node_ptr[l + 1]++; }
        for (int i = 0; i < n_level; ++i) node_ptr[i + 1] += node_ptr[i];
        rows.resize(node_ptr[n_level]);
        std::vector<int> pos(node_ptr.begin(), node_ptr.end() - 1);
        for (int i = 0; i < c.N; ++i) { const int l = nid[i] - off; if (l >= 0 && l < n_level) rows[pos[l]++] = i; }
    }

    // src/thundergbm/tree.cu:85-128 prune_self / try_prune_leaf / reorder_nid
    int try_prune_leaf(int n, int np, std::vector<int> &cnt) {
        const int p = nodes[n].parent_index;
        if (p == -1) return np;
        TreeNode &pn = nodes[p];
        cnt[p]++;
        if (cnt[p] >= 2 && pn.gain < c.p.gamma) {
            nodes[pn.lch_index].is_pruned = true;
            nodes[pn.rch_index].is_pruned = true;
            pn.is_leaf = true;
            return try_prune_leaf(p, np + 2, cnt);
        }
        return np;
    }
    void prune() {
        std::vector<int> cnt(nodes.size(), 0);
        int np = 0;
        for (size_t i = 0; i < nodes.size(); ++i)
            if (nodes[i].is_leaf && nodes[i].is_valid) np = try_prune_leaf((int)i, np, cnt);
        int id = 0;
        for (auto &n : nodes) if (n.is_valid && !n.is_pruned) n.final_id = id++;
    }

    // src/thundergbm/builder/tree_builder.cu:147-194 build_approximate (one tree)
    void build(bool dump_hist) {
        const int d = c.p.depth;
        nid.assign(c.N, 0);
        init_tree();
        gain2.assign(nodes.size(), 0.f);
        level_hist.assign(d, {});
        for (int level = 0; level < d; ++level) {
            const int n_level = 1 << level, off = n_level - 1;
            auto &LH = level_hist[level];
            LH.resize(n_level);
            std::vector<Split> sps(n_level);
            if (level == 0) {
                build_hist(LH[0], nullptr, c.N);
            } else {
                partition_rows(level);
                for (int j = 0; j < n_level / 2; ++j) {
                    const int nl = node_ptr[2 * j + 1] - node_ptr[2 * j], nr = node_ptr[2 * j + 2] - node_ptr[2 * j + 1];
                    if (std::max(nl, nr) == 0) continue;  // :454-465 (no histogram, nodes stay as they are)
                    int comp = 2 * j, sub = 2 * j + 1;
                    if (nl > nr) std::swap(comp, sub);  // :466 build the smaller child, ties -> left
                    build_hist(LH[comp], rows.data() + node_ptr[comp], node_ptr[comp + 1] - node_ptr[comp]);
                    const Hist &par = level_hist[level - 1][j];
                    Hist &S = LH[sub];
                    const int B = (int)c.cut_val.size();
                    S.assign(B);
                    if (c.p.hist_mode == 1) for (int b = 0; b < B; ++b) { S.g[b] = par.g[b] - LH[comp].g[b]; S.h[b] = par.h[b] - LH[comp].h[b]; }
                    else for (int b = 0; b < B; ++b) { S.g[b] = (float)par.g[b] - (float)LH[comp].g[b]; S.h[b] = (float)par.h[b] - (float)LH[comp].h[b]; }
                }
            }
            for (int n = 0; n < n_level; ++n)
                if (!LH[n].g.empty()) {
                    sps[n] = c.p.multi_shards > 0 ? evaluate_multi(LH[n], off + n) : evaluate(LH[n], off + n);
                    gain2[off + n] = sps[n].gain2;
                }
            if (dump_hist) {
                const int B = (int)c.cut_val.size();
                for (int n = 0; n < n_level; ++n)
                    for (int b = 0; b < B; ++b) {
                        const bool have = !LH[n].g.empty();
                        c.hist_dump.push_back(have ? to_f(LH[n].g[b], q.sg) : 0.f);
                        c.hist_dump.push_back(have ? to_f(LH[n].h[b], q.sh) : 0.f);
                    }
            }
            for (int n = 0; n < n_level; ++n) apply(sps[n]);
            if (!move_rows()) break;  // tree_builder.cu:174-181
            if (level >= 2) level_hist[level - 2].clear();
        }
        prune();
    }
};

// src/thundergbm/row_sampler.cu:9-35 do_bagging: M = size of the gradient array (num_class x rows) draws of a uniform
// entry of that array; every entry's (g,h) is multiplied by the number of times it was drawn.  The reference seeds
// thrust's generator from std::rand(); draw j of round r is a counter-based hash here (shared with the CUDA path).
void do_bagging(const Ctx &c, int round, GH *gh) {
    const uint64_t M = (uint64_t)std::max(c.p.num_class, 1) * (uint64_t)c.N;
    std::vector<int> count((size_t)c.K * c.N, 0);
    for (uint64_t j = 0; j < M; ++j) {
        const uint32_t r = mix32(c.p.sample_seed ^ 0xBA661D6Eu, (uint32_t)round, (uint32_t)(j >> 32), (uint32_t)j);
        const uint64_t e = ((uint64_t)r * M) >> 32;
        if (e < (uint64_t)c.K * c.N) count[e]++;
    }
    for (size_t i = 0; i < count.size(); ++i) { gh[i].g = gh[i].g * (float)count[i]; gh[i].h = gh[i].h * (float)count[i]; }
}

// src/thundergbm/builder/shard.cu:8-23 column_sampling, once per round (tree_builder.cu:150-152): max(1, int(F * rate))
// randomly chosen features are put into the ignored set -- the rate is the share that is LEFT OUT.  The reference
// shuffles with std::random_shuffle / rand(); here the features with the smallest hash of (seed, round, feature).
void column_sampling(Ctx &c, int round) {
    c.ignored.clear();
    if (!(c.p.column_sampling_rate < 1.f)) return;
    const int F = c.F, n_ignored = std::min(F, std::max(1, (int)(F * c.p.column_sampling_rate)));
    std::vector<std::pair<uint32_t, int>> key(F);
    for (int f = 0; f < F; ++f) key[f] = {mix32(c.p.sample_seed ^ 0xC01A5EEDu, (uint32_t)round, 0u, (uint32_t)f), f};
    std::sort(key.begin(), key.end());
    c.ignored.assign(F, 0);
    for (int i = 0; i < n_ignored; ++i) c.ignored[key[i].second] = 1;
}

// include/thundergbm/objective/regression_obj.h:35-53 (reg) and :95-114 (binary:logistic)
void init_base_score(Ctx &c, std::vector<GH> &gh) {
    c.base_score = 0;
    const int o = c.p.objective;
    if (!(o == REG_LINEAR || o == REG_LOGISTIC || o == BINARY_LOGISTIC)) return;
    get_gradient(c, 0, c.ypred.data(), gh.data());
    double sg = 0, sh = 0;
    if (c.p.hist_mode == 1) {
        Quant q = choose_quant(c, gh.data(), c.N);
        for (int i = 0; i < c.N; ++i) { sg += quantize(gh[i].g, q.sg, 0xffffffffu, 0, (uint32_t)i, 0); sh += quantize(gh[i].h, q.sh, 0xffffffffu, 0, (uint32_t)i, 1); }
        sg /= q.sg; sh /= q.sh;
    } else {
        for (int i = 0; i < c.N; ++i) { sg += gh[i].g; sh += gh[i].h; }
    }
    const float fg = (float)sg, fh = (float)sh;
    float w = (float)(-(double)fg / fmax((double)fh, 1e-6));
    if (o == BINARY_LOGISTIC) {
        w = 1 / (1 + expf(-w));       // host libm in the reference as well
        w = -logf(1.0f / w - 1.0f);
    }
    c.base_score = w;
    for (int i = 0; i < c.N; ++i) c.ypred[i] = w;
}

// src/thundergbm/metric/*.cu, rank_metric.cpp
float metric(const Ctx &c, const float *yp) {
    const int N = c.N;
    switch (c.p.objective) {
    case REG_LINEAR: case REG_LOGISTIC: {  // pointwise_metric.cu:8-22
        double s = 0;
        for (int i = 0; i < N; ++i) { const float e = yp[i] - c.y[i]; s += (double)(e * e); }
        return sqrtf((float)s / N);
    }
    case BINARY_LOGISTIC: {  // multiclass_metric.cu:33-46
        int ok = 0;
        for (int i = 0; i < N; ++i) { const int k = (1 / (1 + exp(-(double)yp[i])) > 0.5) ? 1 : 0; ok += (float)k == c.y[i]; }
        return 1 - ok / (float)N;
    }
    case MULTI_SOFTMAX: case MULTI_SOFTPROB: {  // multiclass_metric.cu:9-31
        int ok = 0;
        for (int i = 0; i < N; ++i) {
            int mk = 0; float mp = yp[i];
            for (int k = 1; k < c.K; ++k) if (yp[(size_t)k * N + i] > mp) { mp = yp[(size_t)k * N + i]; mk = k; }
            ok += (float)mk == c.y[i];
        }
        return ok / (float)N;
    }
    case RANK_PAIRWISE: case RANK_NDCG: {  // rank_metric.cpp:9-25, 42-66 (MAP), 79-100 (NDCG)
        const int G = (int)c.gptr.size() - 1;
        double sum = 0;  // the reference adds floats in OpenMP reduction order; fixed here: double, group order
        for (int k = 0; k < G; ++k) {
            const int s0 = c.gptr[k], len = c.gptr[k + 1] - s0;
            std::vector<int> idx(len);
            std::iota(idx.begin(), idx.end(), 0);
            const float *sc = yp + s0, *lab = c.y.data() + s0;
            std::stable_sort(idx.begin(), idx.end(), [=](int a, int b) { return sc[a] > sc[b]; });
            if (c.p.objective == RANK_NDCG) {
                if (c.idcg[k] == 0) { sum += 1; continue; }
                float dcg = 0;
                for (int i = 0; i < len; ++i) dcg += discounted_gain((int)lab[idx[i]], i);
                sum += (double)(dcg / c.idcg[k]);
            } else {
                int nh = 0; double ap = 0;
                for (int i = 0; i < len; ++i) if (lab[idx[i]] != 0) { nh++; ap += (double)nh / (i + 1); }
                sum += (double)(nh ? (float)(ap / nh) : 1.f);
            }
        }
        return (float)(sum / (double)G);
    }
    }
    return 0;
}

// src/thundergbm/builder/tree_builder.cu:62-74 predict_in_training; nvcc contracts y += lr*w to one fma
void predict_in_training(const Ctx &c, const Builder &b, float *yp) {
    const float lr = c.p.learning_rate;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < c.N; ++i) {
        int n = b.nid[i];
        while (n != -1 && b.nodes[n].is_pruned) n = b.nodes[n].parent_index;
        yp[i] = fmaf(lr, b.nodes[n].base_weight, yp[i]);
    }
}

void train(Ctx &c) {
    const double t_init = now_s();
#ifdef _OPENMP
    if (c.p.n_threads > 0) omp_set_num_threads(c.p.n_threads);
#endif
    const int o = c.p.objective;
    // src/thundergbm/dataset.cpp:61-64 and trainer.cu:26-37
    c.K = 1;
    if (o == BINARY_LOGISTIC || o == MULTI_SOFTMAX || o == MULTI_SOFTPROB) {
        group_label(c);
        c.p.num_class = (int)c.label.size();
        if (c.p.num_class > 2) c.K = c.p.num_class;
    } else if (o == REG_LINEAR || o == REG_LOGISTIC) c.p.num_class = 1;
    if (o == RANK_NDCG) compute_idcg(c);
    if (c.p.exact_builder) { build_csc(c); c.cut_ptr.assign(c.F + 1, 0); }
    else if (c.p.multi_shards > 0) { find_cuts_multi(c); bin_ids_multi(c); }
    else { find_cuts(c); bin_ids(c); }
    const int N = c.N, K = c.K;
    c.n_nodes = (1 << (c.p.depth + 1)) - 1;
    c.ypred.assign((size_t)K * N, 0.f);
    std::vector<GH> gh((size_t)K * N);
    if (!c.p.exact_builder) init_base_score(c, gh);   // include/thundergbm/booster.h:66-73: only for tree_method = hist
    c.init_seconds = now_s() - t_init;
    const double t0 = now_s();
    for (int r = 0; r < c.p.n_trees; ++r) {  // src/thundergbm/trainer.cu:44-47, include/thundergbm/booster.h:76-93
        const double tr0 = now_s();
        get_gradient(c, r, c.ypred.data(), gh.data());
        if (c.p.bagging) do_bagging(c, r, gh.data());  // include/thundergbm/booster.h:83
        column_sampling(c, r);                         // tree_builder.cu:150-152
        Quant q;
        if (c.p.hist_mode == 1) q = choose_quant(c, gh.data(), (size_t)K * N);
        c.quant_scale.push_back(q.sg); c.quant_scale.push_back(q.sh);
        for (int k = 0; k < K; ++k) {
            q.round = (uint32_t)r; q.k = (uint32_t)k;
            Builder b(c, gh.data() + (size_t)k * N, q);
            if (c.p.exact_builder) b.build_exact();
            else b.build(r == 0 && k == 0 && c.p.keep_nid);
            predict_in_training(c, b, c.ypred.data() + (size_t)k * N);
            c.trees.insert(c.trees.end(), b.nodes.begin(), b.nodes.end());
            c.gain2.insert(c.gain2.end(), b.gain2.begin(), b.gain2.end());
            if (c.p.keep_nid) c.nid_keep.insert(c.nid_keep.end(), b.nid.begin(), b.nid.end());
        }
        c.metric.push_back(metric(c, c.ypred.data()));
        c.round_seconds.push_back(now_s() - tr0);
    }
    c.train_seconds = now_s() - t0;
}

}  // namespace

// =============================================================== C interface (ctypes)
extern "C" {

void *tgo_train(int n_rows, const int *row_ptr, const int *col, const float *val, const float *y, const int *group,
                int n_group, const TgoParam *p) {
    Ctx *c = new Ctx;
    c->p = *p;
    c->N = n_rows;
    const int64_t nnz = row_ptr[n_rows];
    c->row_ptr.assign(row_ptr, row_ptr + n_rows + 1);
    c->col.assign(col, col + nnz);
    c->val.assign(val, val + nnz);
    c->y.assign(y, y + n_rows);
    int F = 0;  // src/thundergbm/dataset.cpp:54-57: n_features = max column index + 1
    for (int64_t i = 0; i < nnz; ++i) F = std::max(F, col[i]);
    c->F = F + 1;
    c->gptr.assign(1, 0);
    for (int i = 0; i < n_group; ++i) c->gptr.push_back(c->gptr.back() + group[i]);
    train(*c);
    return c;
}
void tgo_free(void *h) { delete (Ctx *)h; }
int tgo_n_features(void *h) { return ((Ctx *)h)->F; }
int tgo_n_bins(void *h) { return (int)((Ctx *)h)->cut_val.size(); }
int tgo_num_class(void *h) { return ((Ctx *)h)->p.num_class; }
int tgo_trees_per_round(void *h) { return ((Ctx *)h)->K; }
int tgo_n_nodes(void *h) { return ((Ctx *)h)->n_nodes; }
int tgo_n_labels(void *h) { return (int)((Ctx *)h)->label.size(); }
float tgo_base_score(void *h) { return ((Ctx *)h)->base_score; }
double tgo_train_seconds(void *h) { return ((Ctx *)h)->train_seconds; }
double tgo_init_seconds(void *h) { return ((Ctx *)h)->init_seconds; }
const float *tgo_cut_val(void *h) { return ((Ctx *)h)->cut_val.data(); }
const int *tgo_cut_ptr(void *h) { return ((Ctx *)h)->cut_ptr.data(); }
const int *tgo_bins(void *h) { return ((Ctx *)h)->bin.data(); }
const void *tgo_trees(void *h) { return ((Ctx *)h)->trees.data(); }
const float *tgo_metric(void *h) { return ((Ctx *)h)->metric.data(); }
const float *tgo_ypred(void *h) { return ((Ctx *)h)->ypred.data(); }
const float *tgo_labels(void *h) { return ((Ctx *)h)->label.data(); }
const int *tgo_nid(void *h) { return ((Ctx *)h)->nid_keep.data(); }
const double *tgo_quant_scale(void *h) { return ((Ctx *)h)->quant_scale.data(); }
const float *tgo_gain2(void *h) { return ((Ctx *)h)->gain2.data(); }
const double *tgo_round_seconds(void *h) { return ((Ctx *)h)->round_seconds.data(); }
long tgo_hist_dump_size(void *h) { return (long)((Ctx *)h)->hist_dump.size(); }
const float *tgo_hist_dump(void *h) { return ((Ctx *)h)->hist_dump.data(); }

float tgo_portable_expf(float x) { return portable_expf(x); }

// src/thundergbm/predictor.cu:32-189 predict_raw.  out[t*N+i]; trees [round][class][n_nodes].
// Dense path (F*128*4 <= 48 KB): double accumulator started at base_score, added to a zeroed float.
// CSR path: float accumulator, y += lr*w contracted to fma by nvcc.
void tgo_predict_raw(int n_rows, const int *row_ptr, const int *col, const float *val, int n_features,
                     const void *trees_, int n_rounds, int K, int n_nodes, float lr, float base_score, float *out) {
    const TreeNode *trees = (const TreeNode *)trees_;
    if (K > 1) base_score = 0;
    const bool dense_path = (size_t)n_features * 128 * sizeof(float) <= 48 * 1024;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < n_rows; ++i) {
        const int *ci = col + row_ptr[i];
        const float *vi = val + row_ptr[i];
        const int len = row_ptr[i + 1] - row_ptr[i];
        for (int t = 0; t < K; ++t) {
            double dsum = base_score;
            float fsum = base_score;
            for (int r = 0; r < n_rounds; ++r) {
                const TreeNode *nd = trees + ((size_t)r * K + t) * n_nodes;
                int cur = 0;
                while (!nd[cur].is_leaf) {
                    const int f = nd[cur].split_feature_id;
                    const int *it = std::lower_bound(ci, ci + len, f);
                    // the dense path marks absent features with +inf and tests `fval < INFINITY` (predictor.cu:95-96, :121):
                    // a stored +inf or NaN is taken for absent there; the CSR path compares whatever is stored
                    const bool found = it != ci + len && *it == f && (!dense_path || vi[it - ci] < INFINITY);
                    if (found) cur = vi[it - ci] < nd[cur].split_value ? nd[cur].lch_index : nd[cur].rch_index;
                    else cur = nd[cur].default_right ? nd[cur].rch_index : nd[cur].lch_index;
                }
                const float w = nd[cur].base_weight;
                if (dense_path) dsum += (double)(lr * w); else fsum = fmaf(lr, w, fsum);
            }
            out[(size_t)t * n_rows + i] = dense_path ? (float)(0.0 + dsum) : fsum;
        }
    }
}

// stand-alone pieces for kernel-level parity tests ------------------------------------------
// cut points + global bin ids only
void *tgo_bin_only(int n_rows, const int *row_ptr, const int *col, const float *val, int max_num_bin, int multi_shards) {
    Ctx *c = new Ctx;
    memset(&c->p, 0, sizeof(c->p));
    c->p.max_num_bin = max_num_bin;
    c->p.multi_shards = multi_shards;
    c->N = n_rows;
    const int64_t nnz = row_ptr[n_rows];
    c->row_ptr.assign(row_ptr, row_ptr + n_rows + 1);
    c->col.assign(col, col + nnz);
    c->val.assign(val, val + nnz);
    int F = 0;
    for (int64_t i = 0; i < nnz; ++i) F = std::max(F, col[i]);
    c->F = F + 1;
    if (multi_shards > 0) { find_cuts_multi(*c); bin_ids_multi(*c); }
    else { find_cuts(*c); bin_ids(*c); }
    return c;
}

// gradients for one round from given raw scores (objective as in TgoParam); gh out [K*N][2]
void tgo_gradient(int n_rows, const float *y, const float *yp, int objective, int K, int portable_exp, float *gh_out) {
    Ctx c;
    memset(&c.p, 0, sizeof(c.p));
    c.p.objective = objective; c.p.portable_exp = portable_exp;
    c.N = n_rows; c.K = K;
    c.y.assign(y, y + n_rows);
    get_gradient(c, 0, yp, (GH *)gh_out);
}

}  // extern "C"
