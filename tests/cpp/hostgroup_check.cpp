// Exercises tgbm::HostGroup (the host-side agreement of in-process ranks) with CPU threads: no GPU, no NCCL.
// Prints one line per scenario: "<name> <result of rank 0> <result of rank 1> ..." (1 = all ranks may go on).
#include <cstdio>
#include <thread>
#include <vector>

#include "../../thundergbm_b200/csrc/tgbm_hostgroup.h"

using tgbm::HostGroup;

static void report(const char *name, const std::vector<int> &r) {
    printf("%s", name);
    for (int v : r) printf(" %d", v);
    printf("\n");
}

int main() {
    const int W = 4;
    {   // every rank passes: three rounds in a row succeed
        HostGroup g(W, 5.0);
        std::vector<int> r(W, 1);
        std::vector<std::thread> t;
        for (int k = 0; k < W; ++k) t.emplace_back([&, k] { for (int i = 0; i < 3; ++i) r[k] &= g.agree(true) ? 1 : 0; });
        for (auto &x : t) x.join();
        report("all_ok", r);
    }
    {   // rank 2 fails a local check in the second round: every rank sees the failure in that round and afterwards
        HostGroup g(W, 5.0);
        std::vector<int> first(W), second(W), third(W);
        std::vector<std::thread> t;
        for (int k = 0; k < W; ++k)
            t.emplace_back([&, k] {
                first[k] = g.agree(true);
                second[k] = g.agree(k != 2);
                third[k] = g.agree(true);
            });
        for (auto &x : t) x.join();
        report("one_fails_round1", first);
        report("one_fails_round2", second);
        report("one_fails_round3", third);
    }
    {   // rank 1 raises outside an agreement point and abandons the group: the others are released with a failure
        HostGroup g(W, 30.0);
        std::vector<int> r(W, -1);
        std::vector<std::thread> t;
        for (int k = 0; k < W; ++k)
            t.emplace_back([&, k] {
                if (k == 1) { g.abandon(); return; }
                r[k] = g.agree(true);
            });
        for (auto &x : t) x.join();
        report("abandon", r);
    }
    {   // rank 3 never arrives: the time limit ends the wait of the others
        HostGroup g(W, 0.3);
        std::vector<int> r(W, -1);
        std::vector<std::thread> t;
        for (int k = 0; k < W - 1; ++k) t.emplace_back([&, k] { r[k] = g.agree(true); });
        for (auto &x : t) x.join();
        report("missing_rank", r);
    }
    return 0;
}
