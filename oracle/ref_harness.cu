// Golden-vector harness: drives the reference's own classes (public headers of
// the reference tree, linked against the reference library built by
// oracle/build_ref.sh) on a binary CSR input and dumps what the parity tests
// pin: cut points, global bin ids, the trained model file, raw predictions on
// the training rows and the per-round metric log (stdout).
//
// Test infrastructure only; never linked into or called by the product.
//
// usage: ref_harness <input.tgbin> <out_dir> [key=value ...]
//   keys: depth n_trees max_num_bin lambda gamma min_child_weight learning_rate
//         objective tree_method verbose n_device dump_bins
//   n_device > 1 (the reference's column-sharded HistTreeBuilder): dump_bins=1, the default, writes the devices' cut
//   points and bin matrices and stops; dump_bins=0 trains.
// input.tgbin: i32 n_rows, i32 n_group, i64 nnz, i32 row_ptr[n_rows+1],
//              i32 col[nnz], f32 val[nnz], f32 y[n_rows], i32 group[n_group]
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#include <fstream>
#include <map>
#include <memory>
#include <chrono>
#include <sstream>
#include <iostream>
#include <mutex>

#define private public
#define protected public
#include <thundergbm/builder/hist_tree_builder_single.h>
#include <thundergbm/builder/hist_tree_builder.h>
#undef private
#undef protected
#include <thundergbm/trainer.h>
#include <thundergbm/parser.h>
#include <thundergbm/predictor.h>
#include <thundergbm/dataset.h>

template <typename T>
static void dump(const std::string &path, const T *p, size_t n) {
    FILE *f = fopen(path.c_str(), "wb");
    if (!f) { perror(path.c_str()); exit(2); }
    fwrite(p, sizeof(T), n, f);
    fclose(f);
}

int main(int argc, char **argv) {
    if (argc < 3) { fprintf(stderr, "usage: ref_harness in.tgbin out_dir [k=v]\n"); return 1; }
    std::string in = argv[1], out = argv[2];
    GBMParam p;
    p.depth = 6; p.n_trees = 40; p.n_device = 1; p.min_child_weight = 1; p.lambda = 1; p.gamma = 1;
    p.rt_eps = 1e-6; p.max_num_bin = 255; p.verbose = 1; p.profiling = false; p.column_sampling_rate = 1;
    p.bagging = false; p.n_parallel_trees = 1; p.learning_rate = 1; p.objective = "reg:linear";
    p.num_class = 1; p.tree_method = "hist"; p.tree_per_rounds = 1;
    bool dump_bins = true;
    for (int i = 3; i < argc; ++i) {
        char k[256], v[256];
        if (sscanf(argv[i], "%[^=]=%s", k, v) != 2) continue;
        std::string key(k);
        if (key == "depth") p.depth = atoi(v);
        else if (key == "n_trees") p.n_trees = atoi(v);
        else if (key == "max_num_bin") p.max_num_bin = atoi(v);
        else if (key == "lambda") p.lambda = atof(v);
        else if (key == "gamma") p.gamma = atof(v);
        else if (key == "min_child_weight") p.min_child_weight = atof(v);
        else if (key == "learning_rate") p.learning_rate = atof(v);
        else if (key == "objective") p.objective = v;
        else if (key == "tree_method") p.tree_method = v;
        else if (key == "verbose") p.verbose = atoi(v);
        else if (key == "num_class") p.num_class = atoi(v);
        else if (key == "dump_bins") dump_bins = atoi(v);
        else if (key == "n_device") p.n_device = atoi(v);  // > 1: the reference's column-sharded HistTreeBuilder
    }
    el::Loggers::reconfigureAllLoggers(el::ConfigurationType::Format, "%level : %msg");
    el::Loggers::reconfigureAllLoggers(el::Level::Debug, el::ConfigurationType::Enabled, "false");
    el::Loggers::reconfigureAllLoggers(el::Level::Trace, el::ConfigurationType::Enabled, "false");
    el::Loggers::reconfigureAllLoggers(el::ConfigurationType::PerformanceTracking, "false");

    FILE *f = fopen(in.c_str(), "rb");
    if (!f) { perror(in.c_str()); return 2; }
    int n_rows, n_group; long long nnz;
    if (fread(&n_rows, 4, 1, f) != 1 || fread(&n_group, 4, 1, f) != 1 || fread(&nnz, 8, 1, f) != 1) return 2;
    std::vector<int> row_ptr(n_rows + 1), col(nnz), group(n_group);
    std::vector<float> val(nnz), y(n_rows);
    size_t got = 0;
    got += fread(row_ptr.data(), 4, n_rows + 1, f);
    got += fread(col.data(), 4, nnz, f);
    got += fread(val.data(), 4, nnz, f);
    got += fread(y.data(), 4, n_rows, f);
    got += fread(group.data(), 4, n_group, f);
    fclose(f);
    if (got != (size_t)(n_rows + 1) + 2 * (size_t)nnz + n_rows + n_group) { fprintf(stderr, "short read\n"); return 2; }

    DataSet ds;
    ds.load_from_sparse(n_rows, val.data(), row_ptr.data(), col.data(), y.data(), group.data(), n_group, p);

    if (dump_bins && p.n_device == 1) {
        // what the reference's 1-GPU builder computes at init: cut points and global bin ids
        GBMParam q = p;
        if (q.objective.find("multi:") != std::string::npos || q.objective.find("binary:") != std::string::npos)
            q.num_class = ds.label.size();
        HistTreeBuilder_single b;
        b.init(ds, q);
        auto &cut = b.cut[0];
        int B = cut.cut_points_val.size();
        dump(out + "/cut_val.f32", cut.cut_points_val.host_data(), B);
        dump(out + "/cut_row_ptr.i32", cut.cut_row_ptr.host_data(), cut.cut_row_ptr.size());
        dump(out + "/cut_fid.i32", cut.cut_fid.host_data(), B);
        dump(out + "/csr_bin_id.i32", b.csr_bin_id[0].host_data(), b.csr_bin_id[0].size());
        printf("HARNESS n_bins %d nnz %lld n_features %zu\n", B, nnz, ds.n_features());
    }

    if (dump_bins && p.n_device > 1) {
        // what the reference's column-sharded builder computes at init, per device: cut points (descending
        // within a feature) and the dense matrix of local bin ids (missing = max_num_bin).  A run of its own: a second
        // multi-device builder in the process disturbs the reference's training (it aborts in SyncMem or loses
        // histogram updates), and one made after the training computes other cut points for some columns.
        GBMParam q = p;
        if (q.objective.find("multi:") != std::string::npos || q.objective.find("binary:") != std::string::npos)
            q.num_class = ds.label.size();
        HistTreeBuilder b;
        b.init(ds, q);
        for (int d = 0; d < p.n_device; ++d) {
            auto &cut = b.cut[d];
            std::string sfx = "_d" + std::to_string(d);
            dump(out + "/cut_val" + sfx + ".f32", cut.cut_points_val.host_data(), cut.cut_points_val.size());
            dump(out + "/cut_row_ptr" + sfx + ".i32", cut.cut_row_ptr.host_data(), cut.cut_row_ptr.size());
            dump(out + "/dense_bin_id" + sfx + ".u8", b.dense_bin_id[d].host_data(), b.dense_bin_id[d].size());
            printf("HARNESS device %d n_bins %zu n_column %d column_offset %d\n", d, cut.cut_points_val.size(),
                   b.shards[d].columns.n_column, b.shards[d].columns.column_offset);
        }
        printf("HARNESS dump only\n");
        return 0;
    }

    TreeTrainer trainer;
    auto t0 = std::chrono::high_resolution_clock::now();
    std::vector<std::vector<Tree>> model = trainer.train(p, ds);
    auto t1 = std::chrono::high_resolution_clock::now();
    printf("HARNESS train_wall_s %.6f base_score %.9g num_class %d tree_per_rounds %d\n",
           std::chrono::duration<double>(t1 - t0).count(), p.base_score, p.num_class, p.tree_per_rounds);
    Parser parser;
    parser.save_model(out + "/tgbm.model", p, model, ds);

    Predictor pred;
    SyncArray<float_type> yp;
    pred.predict_raw(p, model, ds, yp);
    dump(out + "/raw_pred.f32", yp.host_data(), yp.size());
    printf("HARNESS done raw_pred %zu\n", yp.size());
    return 0;
}
