// thundergbm-train <conf> [key=value ...]  -- same contract as the reference's CLI
// (src/thundergbm/thundergbm_train.cpp:10-40): parse the conf, load the LibSVM file named by `data=`,
// train, write ./tgbm.model.
#include <chrono>
#include <cstdio>

#include "../tgbm_booster.h"

int main(int argc, char **argv) {
    using namespace tgbm;
    if (argc < 2) {
        printf("Usage: <config>\n");
        return 0;
    }
    try {
        GBMParam p;
        parse_param(p, argc, argv);
        set_verbosity(p.verbose);
        DataSet ds;
        ds.load_from_file(p.path, p);
        if (p.tree_method == "auto") p.tree_method = ds.n_features > 20000 ? "exact" : "hist";
        TGBM_CHECK(p.tree_method == "hist", "only tree_method=hist is implemented (auto picks exact above 20000 features)");
        TGBM_CHECK(p.n_device == 1, "n_gpus > 1: launch one process per GPU through the library's booster interface");
        Booster booster(p, nullptr);
        booster.init(ds);
        const auto t0 = std::chrono::high_resolution_clock::now();
        booster.boost(p.n_trees);
        booster.sync();
        const auto t1 = std::chrono::high_resolution_clock::now();
        const auto metrics = booster.get_metrics();
        const char *name = metric_name(objective_from_name(p.objective));
        for (size_t i = 0; i < metrics.size(); ++i) log_info("[%zu/%d] %s = %g", i + 1, p.n_trees, name, metrics[i]);
        log_info("training time = %g", std::chrono::duration<float>(t1 - t0).count());
        p.base_score = booster.base_score();
        p.num_class = booster.num_class();
        auto model = booster.get_model();
        save_model("tgbm.model", p, model, ds.label);
    } catch (const std::exception &e) {
        fprintf(stderr, "thundergbm-train: %s\n", e.what());
        return 1;
    }
    return 0;
}
