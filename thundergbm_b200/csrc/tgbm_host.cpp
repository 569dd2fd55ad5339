// Host side of the drop-in boundary: data-set containers, .conf/argv parser,
// binary model file, logging.  Mirrors the behaviour of the reference's
// dataset.cpp, parser.cpp and logger configuration for the histogram path.
#include "tgbm_common.h"

#include <algorithm>
#include <cstdarg>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <thread>

namespace tgbm {

static int g_verbose = 1;
void set_verbosity(int v) { g_verbose = v; }
int verbosity() { return g_verbose; }
void log_info(const char *fmt, ...) {
    if (g_verbose < 1) return;
    va_list ap;
    va_start(ap, fmt);
    vfprintf(stdout, fmt, ap);
    va_end(ap);
    fputc('\n', stdout);
    fflush(stdout);
}

// src/thundergbm/dataset.cpp:20-69.  The CSR arrays are copied; n_features = max column + 1;
// classification objectives regroup the labels; ranking objectives take the query group sizes.
void DataSet::load_from_sparse(int n, const float *v, const int *rp, const int *ci, const float *yy, const int *grp,
                               int num_group, GBMParam &param, bool lazy) {
    TGBM_CHECK(n >= 0 && rp != nullptr, "bad CSR input");
    const long long nnz = rp[n];
    TGBM_CHECK(nnz >= 0, "bad CSR row_ptr");
    n_rows = n;
    row_ptr.clear(); col.clear(); val.clear();
    this->rp = rp; this->ci = ci; this->vv = v;  // borrowed: the 2.4 GB of a Higgs-sized CSR are not copied on the host
    const bool borrow = lazy && yy != nullptr;
    y.clear();
    if (!borrow) { if (yy) y.assign(yy, yy + n); else y.assign(n, 0.f); }
    yv = borrow ? yy : y.data();
    labels_raw = false;
    label.clear();
    group.clear();
    // n_features = largest column index + 1 (dataset.cpp:54-57), scanned by a few threads
    n_features = -1;
    if (!lazy) n_features = count_features();
    const int o = objective_from_name(param.objective);
    if (yy && need_group_label(o)) {
        if (borrow) { distinct_labels(yy, (size_t)n); labels_raw = true; }
        else group_label();
        param.num_class = (int)label.size();
    }
    if (need_group_file(o))
        for (int i = 0; i < num_group; ++i) group.push_back(grp[i]);
}

int DataSet::count_features() const {
    const long long nnz = rp ? rp[n_rows] : 0;
    const int nt = (int)std::max<long long>(1, std::min<long long>(16, nnz / (1 << 22)));
    std::vector<int> part(nt, -1);
    std::vector<std::thread> th;
    for (int t = 0; t < nt; ++t)
        th.emplace_back([&, t] {
            const long long a = nnz * t / nt, b = nnz * (t + 1) / nt;
            int m = -1;
            for (long long i = a; i < b; ++i) m = std::max(m, ci[i]);
            part[t] = m;
        });
    for (auto &x : th) x.join();
    return *std::max_element(part.begin(), part.end()) + 1;
}

// src/thundergbm/dataset.cpp:83-101: labels cast to int, sorted, uniqued; y -> index of its value
void DataSet::distinct_labels(const float *yy, size_t n) {
    // distinct int(label) values, found by a few threads; a thread keeps what it has seen in a small unsorted array
    // (two or a handful of classes is the rule) and falls back to a sorted vector beyond that
    const int nt = (int)std::max<size_t>(1, std::min<size_t>(16, n / (1 << 20)));
    std::vector<std::vector<int>> found(nt);
    {
        std::vector<std::thread> th;
        for (int t = 0; t < nt; ++t)
            th.emplace_back([&, t] {
                int small[16], ns = 0;
                std::vector<int> &big = found[t];
                for (size_t i = n * t / nt; i < n * (t + 1) / nt; ++i) {
                    const int v = (int)yy[i];
                    bool hit = false;
                    for (int k = 0; k < ns; ++k) hit |= small[k] == v;
                    if (hit) continue;
                    if (ns < 16) { small[ns++] = v; continue; }
                    auto it = std::lower_bound(big.begin(), big.end(), v);
                    if (it == big.end() || *it != v) big.insert(it, v);
                }
                big.insert(big.end(), small, small + ns);
            });
        for (auto &x : th) x.join();
    }
    std::vector<int> t;
    for (auto &f : found) t.insert(t.end(), f.begin(), f.end());
    std::sort(t.begin(), t.end());
    t.erase(std::unique(t.begin(), t.end()), t.end());
    label.clear();
    for (int v : t) label.push_back((float)v);
}

void DataSet::group_label() {
    const size_t n = y.size();
    distinct_labels(y.data(), n);
    const int nt = (int)std::max<size_t>(1, std::min<size_t>(16, n / (1 << 20)));
    // y -> index of its value among the labels; a label that is not an integer maps to 0
    const int nl = (int)label.size();
    std::vector<std::thread> th;
    for (int k = 0; k < nt; ++k)
        th.emplace_back([&, k] {
            for (size_t i = n * k / nt; i < n * (k + 1) / nt; ++i) {
                const float v = y[i];
                int idx = 0;
                if (nl <= 16) {
                    for (int j = 0; j < nl; ++j) idx = label[j] == v ? j : idx;
                } else {
                    auto it = std::lower_bound(label.begin(), label.end(), v);
                    idx = (it != label.end() && *it == v) ? (int)(it - label.begin()) : 0;
                }
                y[i] = (float)idx;
            }
        });
    for (auto &x : th) x.join();
}

// src/thundergbm/dataset.cpp:71-81
void DataSet::load_group_file(const std::string &file) {
    std::ifstream ifs(file);
    TGBM_CHECK(ifs.is_open(), "ranking objective needs a group file, not found: " + file);
    group.clear();
    int g;
    while (ifs >> g) group.push_back(g);
    log_info("#groups = %zu", group.size());
}

// src/thundergbm/dataset.cpp:106-320: LibSVM text, `label idx:val ...`, 1-based idx, '#' comments.
// The buffer is cut at line ends into one piece per thread; the pieces are parsed independently and joined in order.
namespace {
struct SvmPiece {
    std::vector<float> y, val;
    std::vector<int> col, row_nnz;
    int maxf = 0;
};
// atof for the common short decimals: up to 15 digits and a power of ten up to 22 are exact in double, so one
// multiplication or division gives the correctly rounded value (Clinger's fast path) -- the same double atof
// returns.  Anything else (long mantissas, large exponents, inf/nan spellings) goes to atof itself.
double fast_atof(const char *q, const char *stop) {
    static const double p10[] = {1e0, 1e1, 1e2, 1e3, 1e4, 1e5, 1e6, 1e7, 1e8, 1e9, 1e10, 1e11,
                                 1e12, 1e13, 1e14, 1e15, 1e16, 1e17, 1e18, 1e19, 1e20, 1e21, 1e22};
    const char *c = q;
    bool neg = false;
    if (c < stop && (*c == '+' || *c == '-')) { neg = *c == '-'; ++c; }
    unsigned long long m = 0;
    int digits = 0, frac = 0;
    bool any = false;
    while (c < stop && *c >= '0' && *c <= '9') { m = m * 10 + (unsigned)(*c - '0'); digits += (m != 0); any = true; ++c; if (digits > 15) return atof(q); }
    if (c < stop && *c == '.') {
        ++c;
        while (c < stop && *c >= '0' && *c <= '9') { m = m * 10 + (unsigned)(*c - '0'); digits += (m != 0); ++frac; any = true; ++c; if (digits > 15) return atof(q); }
    }
    if (!any) return atof(q);
    int ex = 0;
    if (c < stop && (*c == 'e' || *c == 'E')) {
        ++c;
        bool eneg = false;
        if (c < stop && (*c == '+' || *c == '-')) { eneg = *c == '-'; ++c; }
        if (!(c < stop && *c >= '0' && *c <= '9')) return atof(q);
        while (c < stop && *c >= '0' && *c <= '9') { ex = ex * 10 + (*c - '0'); ++c; if (ex > 400) return atof(q); }
        if (eneg) ex = -ex;
    }
    if (c < stop && (*c == '+' || *c == '-' || *c == '.' || *c == 'e' || *c == 'E' || *c == 'x' || *c == 'X' || *c == 'p' || *c == 'P'))
        return atof(q);  // odd token (or a hex float): let atof decide
    const int e10 = ex - frac;
    if (e10 < -22 || e10 > 22) return atof(q);
    double v = (double)m;
    v = e10 < 0 ? v / p10[-e10] : v * p10[e10];
    return neg ? -v : v;
}

void parse_svm_piece(const char *p, const char *end, SvmPiece &o) {
    auto is_num = [](char c) { return (c >= '0' && c <= '9') || c == '+' || c == '-' || c == '.' || c == 'e' || c == 'E'; };
    while (p < end) {
        const char *le = p;
        while (le < end && *le != '\n' && *le != '\r' && *le != '\0') ++le;
        const char *q = p;
        const char *stop = le;
        for (const char *c = p; c < le; ++c) if (*c == '#') { stop = c; break; }
        while (q < stop && !is_num(*q)) ++q;
        if (q < stop) {
            o.y.push_back((float)fast_atof(q, stop));
            const size_t before = o.col.size();
            while (q < stop && is_num(*q)) ++q;
            while (q < stop) {
                while (q < stop && !is_num(*q)) ++q;
                if (q >= stop) break;
                const char *a = q;
                while (q < stop && is_num(*q)) ++q;
                const char *c = q;
                while (c < stop && (*c == ' ' || *c == '\t')) ++c;
                if (c < stop && *c == ':') {
                    const int fid = atoi(a);
                    q = c + 1;
                    while (q < stop && !is_num(*q)) ++q;
                    const float fv = (float)fast_atof(q, stop);
                    while (q < stop && is_num(*q)) ++q;
                    if (fid >= 1) {  // LibSVM indices are 1-based; 0 or a negative index names no column and is dropped
                        o.col.push_back(fid - 1);
                        o.val.push_back(fv);
                        o.maxf = std::max(o.maxf, fid);
                    }
                }
            }
            o.row_nnz.push_back((int)(o.col.size() - before));
        }
        p = le + 1;
    }
}
}  // namespace

void DataSet::load_from_file(const std::string &file, GBMParam &param) {
    std::ifstream ifs(file, std::ifstream::binary | std::ifstream::ate);
    TGBM_CHECK(ifs.is_open(), "file not found: " + file);
    std::string buf((size_t)std::max<std::streamoff>(0, ifs.tellg()), '\0');
    ifs.seekg(0);
    ifs.read(&buf[0], (std::streamsize)buf.size());
    buf.resize((size_t)std::max<std::streamsize>(0, ifs.gcount()));
    row_ptr.assign(1, 0);
    col.clear(); val.clear(); y.clear(); label.clear(); group.clear();
    const char *base = buf.data(), *end = base + buf.size();
    const int nt = (int)std::max<size_t>(1, std::min<size_t>(16, buf.size() / (4u << 20)));
    std::vector<const char *> cut(nt + 1, end);
    cut[0] = base;
    for (int t = 1; t < nt; ++t) {
        const char *c = base + buf.size() * t / nt;
        c = std::max(c, cut[t - 1]);
        while (c < end && *c != '\n') ++c;
        cut[t] = c < end ? c + 1 : end;
    }
    std::vector<SvmPiece> piece(nt);
    {
        std::vector<std::thread> th;
        for (int t = 0; t < nt; ++t) th.emplace_back([&, t] { parse_svm_piece(cut[t], cut[t + 1], piece[t]); });
        for (auto &x : th) x.join();
    }
    int maxf = 0;
    for (auto &pc : piece) {
        y.insert(y.end(), pc.y.begin(), pc.y.end());
        col.insert(col.end(), pc.col.begin(), pc.col.end());
        val.insert(val.end(), pc.val.begin(), pc.val.end());
        for (int c : pc.row_nnz) row_ptr.push_back(row_ptr.back() + c);
        maxf = std::max(maxf, pc.maxf);
    }
    n_rows = (int)y.size();
    n_features = maxf;
    rp = row_ptr.data(); ci = col.data(); vv = val.data(); yv = y.data();
    labels_raw = false;
    log_info("#instances = %d, #features = %d", n_rows, n_features);
    const int o = objective_from_name(param.objective);
    if (need_group_file(o)) load_group_file(file + ".group");
    if (need_group_label(o)) {
        group_label();
        param.num_class = (int)label.size();
    }
}

// src/thundergbm/parser.cpp:9-100: defaults, then `key=value` lines of the conf file, then argv.
void parse_param(GBMParam &mp, int argc, char **argv) {
    mp = GBMParam();
    mp.hist_mode = default_hist_mode();  // TGBM_HIST_MODE, else fp32; the conf key hist_mode overrides it
    auto parse_value = [&](const char *name_val) {
        char name[256], val[256];
        if (sscanf(name_val, "%255[^=]=%255s", name, val) != 2) return;
        const std::string k(name);
        if (k == "max_depth" || k == "depth") mp.depth = atoi(val);
        else if (k == "num_round" || k == "n_trees") mp.n_trees = atoi(val);
        else if (k == "n_gpus") mp.n_device = atoi(val);
        else if (k == "verbosity" || k == "verbose") mp.verbose = atoi(val);
        else if (k == "profiling") mp.profiling = atoi(val);
        else if (k == "data") mp.path = val;
        else if (k == "max_bin" || k == "max_num_bin") mp.max_num_bin = atoi(val);
        else if (k == "colsample" || k == "column_sampling_rate") mp.column_sampling_rate = (float)atof(val);
        else if (k == "bagging") mp.bagging = atoi(val);
        else if (k == "num_parallel_tree" || k == "n_parallel_trees") mp.n_parallel_trees = atoi(val);
        else if (k == "eta" || k == "learning_rate") mp.learning_rate = (float)atof(val);
        else if (k == "objective") mp.objective = val;
        else if (k == "num_class") mp.num_class = atoi(val);
        else if (k == "min_child_weight") mp.min_child_weight = (float)atoi(val);  // atoi, as in the reference
        else if (k == "lambda" || k == "lambda_tgbm") mp.lambda = (float)atof(val);
        else if (k == "gamma" || k == "min_split_loss") mp.gamma = (float)atof(val);
        else if (k == "tree_method") mp.tree_method = val;
        else if (k == "quant_bits") mp.quant_bits = atoi(val);
        else if (k == "hist_mode") mp.hist_mode = hist_mode_from_name(val);
        else if (k == "column_shards") mp.column_shards = atoi(val);
        else if (k == "seed" || k == "sample_seed") mp.sample_seed = (unsigned)strtoul(val, nullptr, 10);
        else log_info("\"%s\" is unknown option!", name);
    };
    if (argc >= 2) {
        std::ifstream conf(argv[1]);
        std::string line;
        while (std::getline(conf, line)) parse_value(line.c_str());
    }
    for (int i = 0; i < argc; ++i) parse_value(argv[i]);
}

// src/thundergbm/parser.cpp:146-171 -- little-endian native dump:
// i32 len, objective, f32 lr, i32 num_class, i32 n_trees, f32 base_score, i32 n_label, f32 label[],
// i32 n_rounds, { i32 n_k, { u64 n_nodes, TreeNode[n_nodes] } x n_k } x n_rounds
void save_model(const std::string &path, const GBMParam &p, const std::vector<std::vector<Tree>> &model,
                const std::vector<float> &label) {
    std::ofstream out(path, std::ios::binary);
    TGBM_CHECK(out.is_open(), "cannot write model file " + path);
    const int len = (int)p.objective.size();
    out.write((const char *)&len, 4);
    out.write(p.objective.data(), len);
    out.write((const char *)&p.learning_rate, 4);
    out.write((const char *)&p.num_class, 4);
    out.write((const char *)&p.n_trees, 4);
    out.write((const char *)&p.base_score, 4);
    const int nl = (int)label.size();
    out.write((const char *)&nl, 4);
    out.write((const char *)label.data(), 4 * (size_t)nl);
    const int nr = (int)model.size();
    out.write((const char *)&nr, 4);
    for (const auto &round : model) {
        const int nk = (int)round.size();
        out.write((const char *)&nk, 4);
        for (const auto &t : round) {
            const uint64_t nn = t.nodes.size();
            out.write((const char *)&nn, 8);
            out.write((const char *)t.nodes.data(), sizeof(TreeNode) * nn);
        }
    }
}

// src/thundergbm/parser.cpp:102-145
void load_model(const std::string &path, GBMParam &p, std::vector<std::vector<Tree>> &model, std::vector<float> &label) {
    std::ifstream in(path, std::ios::binary);
    TGBM_CHECK(in.is_open(), "cannot read model file " + path);
    int len = 0;
    in.read((char *)&len, 4);
    TGBM_CHECK(len >= 0 && len < 4096, "corrupt model file");
    std::string obj(len, '\0');
    in.read(&obj[0], len);
    p.objective = obj;
    in.read((char *)&p.learning_rate, 4);
    in.read((char *)&p.num_class, 4);
    in.read((char *)&p.n_trees, 4);
    in.read((char *)&p.base_score, 4);
    int nl = 0;
    in.read((char *)&nl, 4);
    TGBM_CHECK(nl >= 0 && nl < (1 << 24), "corrupt model file");
    label.resize(nl);
    in.read((char *)label.data(), 4 * (size_t)nl);
    int nr = 0;
    in.read((char *)&nr, 4);
    TGBM_CHECK(nr >= 0 && nr < (1 << 24), "corrupt model file");
    model.clear();
    for (int r = 0; r < nr; ++r) {
        int nk = 0;
        in.read((char *)&nk, 4);
        TGBM_CHECK(nk >= 0 && nk < (1 << 20), "corrupt model file");
        std::vector<Tree> v(nk);
        for (auto &t : v) {
            uint64_t nn = 0;
            in.read((char *)&nn, 8);
            TGBM_CHECK(nn < (1ull << 28), "corrupt model file");
            t.nodes.resize(nn);
            in.read((char *)t.nodes.data(), sizeof(TreeNode) * nn);
        }
        model.push_back(std::move(v));
    }
    TGBM_CHECK(bool(in), "truncated model file " + path);
}

}  // namespace tgbm
