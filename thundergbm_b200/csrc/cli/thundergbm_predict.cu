// thundergbm-predict <conf>  -- src/thundergbm/thundergbm_predict.cpp:11-41: reads ./tgbm.model and the
// LibSVM file named by `data=`, logs the objective's default metric on it.
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
        std::vector<std::vector<Tree>> model;
        std::vector<float> label;
        load_model("tgbm.model", p, model, label);
        DataSet ds;
        ds.load_from_file(p.path, p);
        std::vector<float> y;
        predict_raw(ds, model, p.learning_rate, p.base_score, y);
        const int o = objective_from_name(p.objective);
        log_info("%s = %g", metric_name(o), metric_score(o, ds, p.num_class, y));
        predict_transform(o, p.num_class, label, ds.n_rows, y);
    } catch (const std::exception &e) {
        fprintf(stderr, "thundergbm-predict: %s\n", e.what());
        return 1;
    }
    return 0;
}
