// thundergbm-train <conf> [key=value ...]  -- same contract as the reference's CLI
// (src/thundergbm/thundergbm_train.cpp:10-40): parse the conf, load the LibSVM file named by `data=`,
// train, write ./tgbm.model.
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
        auto model = train_model(p, ds);  // n_gpus > 1: one host thread per GPU, rows sharded
        save_model("tgbm.model", p, model, ds.label);
    } catch (const std::exception &e) {
        fprintf(stderr, "thundergbm-train: %s\n", e.what());
        return 1;
    }
    return 0;
}
