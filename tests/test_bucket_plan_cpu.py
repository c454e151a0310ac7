"""The planner that orders the flat layout by the point at which backward is finished
with each tensor and cuts the optimizer step into buckets
(saga_b200/host/b200_adam_op.hpp: b200_plan_buckets), on CPU with made-up programs."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r'''
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>
#include "b200_adam_op.hpp"

using namespace saga;

#define CHECK(c) do { if(!(c)) { printf("line %d: %s\n", __LINE__, #c); return 1; } } while(0)

static size_t padded(size_t n) { return (n + 15) / 16 * 16; }

// every element covered exactly once, buckets consecutive, anchors never decreasing
static int well_formed(const std::vector<B200PlanEntry> &e, const B200Plan &p)
{
    size_t total[2] = {0, 0}, at[2] = {0, 0};
    for(auto &x : e)
        total[x.dtype] += padded(x.elements);
    CHECK(p.order[0].size() + p.order[1].size() == e.size());
    CHECK(p.buckets.size() == p.anchors.size() && !p.buckets.empty());
    for(size_t b = 0; b < p.buckets.size(); b++) {
        CHECK(p.buckets[b].half_first == at[0] && p.buckets[b].float_first == at[1]);
        at[0] += p.buckets[b].half_count;
        at[1] += p.buckets[b].float_count;
        if(b)
            CHECK(p.anchors[b] >= p.anchors[b - 1]);
    }
    CHECK(at[0] == total[0] && at[1] == total[1]);
    return 0;
}

int main()
{
    // a 4-layer net: forward ops 0..3 read w, backward ops 4..11 come in reverse layer
    // order; each layer has a big fp16 weight and a small fp32 pair.  Reference order =
    // layer order, i.e. the reverse of the order in which backward finishes with them.
    std::vector<B200PlanEntry> e;
    const size_t sizes[4] = {1000, 40000, 40000, 20000};
    for(int l = 0; l < 4; l++) {
        const long last = 4 + 2 * (3 - l) + 1;   // layer 3 is final first
        e.push_back({B200OPT_HALF, sizes[l], last});
        e.push_back({B200OPT_FLOAT, 64, last - 1});
    }
    {
        B200Plan p = b200_plan_buckets(e, 3, true);
        if(well_formed(e, p))
            return 1;
        // backward order: layer 3 first, layer 0 last, in both groups
        CHECK(p.order[B200OPT_HALF] == (std::vector<size_t>{6, 4, 2, 0}));
        CHECK(p.order[B200OPT_FLOAT] == (std::vector<size_t>{7, 5, 3, 1}));
        CHECK(p.buckets.size() == 3);
        // cuts fall where the running size is closest to a third and two thirds of the
        // total; a bucket follows the last op that touches any of its tensors (the fp32
        // pair of layer 2, final at op 6, still fits the first bucket)
        CHECK(p.anchors[0] == 6 && p.anchors[1] == 8 && p.anchors[2] == 11);
        CHECK(p.buckets[0].half_count == padded(20000) && p.buckets[1].half_count == padded(40000));
        CHECK(p.buckets[2].half_count == padded(40000) + padded(1000));
        CHECK(p.buckets[0].float_count == 128 && p.buckets[1].float_count == 64 &&
              p.buckets[2].float_count == 64);
    }
    {
        // the reference's order kept: a bucket waits for the latest of its members, so the
        // first bucket (layers 0 and 1) can only go at the very end
        B200Plan p = b200_plan_buckets(e, 2, false);
        if(well_formed(e, p))
            return 1;
        CHECK(p.order[B200OPT_HALF] == (std::vector<size_t>{0, 2, 4, 6}));
        CHECK(p.buckets.size() == 2 && p.anchors[0] == 11 && p.anchors[1] == 11);
    }
    {
        // one bucket, more buckets than tensors, nothing to train
        B200Plan one = b200_plan_buckets(e, 1, true);
        CHECK(one.buckets.size() == 1 && one.buckets[0].half_count == padded(1000) + 2 * padded(40000) + padded(20000));
        B200Plan many = b200_plan_buckets(e, 64, true);
        if(well_formed(e, many))
            return 1;
        CHECK(many.buckets.size() <= e.size());
        B200Plan none = b200_plan_buckets({}, 4, true);
        CHECK(none.buckets.size() == 1 && none.buckets[0].half_count == 0);
    }
    {
        // tensors that one op finishes together are never split; a tensor no op touches
        // (last_touch -1) sorts first and its bucket still gets a usable anchor
        std::vector<B200PlanEntry> f = {{B200OPT_HALF, 5000, 9}, {B200OPT_HALF, 5000, 9},
                                        {B200OPT_HALF, 5000, 9}, {B200OPT_HALF, 100, -1},
                                        {B200OPT_HALF, 5000, 3}};
        B200Plan p = b200_plan_buckets(f, 4, true);
        if(well_formed(f, p))
            return 1;
        CHECK(p.order[B200OPT_HALF] == (std::vector<size_t>{3, 4, 0, 1, 2}));
        CHECK(p.buckets.size() == 2 && p.anchors[0] == 3 && p.anchors[1] == 9);
        CHECK(p.buckets[1].half_count == 3 * padded(5000));
    }
    {
        // a big tensor at the end of the reference order still leaves two buckets
        std::vector<B200PlanEntry> f = {{B200OPT_HALF, 100, 7}, {B200OPT_HALF, 100, 6},
                                        {B200OPT_HALF, 90000, 5}};
        B200Plan p = b200_plan_buckets(f, 2, false);
        if(well_formed(f, p))
            return 1;
        CHECK(p.buckets.size() == 2 && p.buckets[1].half_count == padded(90000));
    }
    {
        // placement in the op list: ops are strings, buckets are "B<k>@<anchor>", "END" closes
        // the step; they arrive at the end of the list in bucket order
        std::vector<std::string> ops = {"f0", "f1", "b1", "b0", "B0@b1", "B1@b1", "B2@b0", "B3@gone", "END"};
        auto is_bucket = [](const std::string &s) { return s[0] == 'B'; };
        auto anchor_of = [](const std::string &s) { return s.substr(s.find('@') + 1); };
        auto is_final = [](const std::string &s) { return s == "END"; };
        b200_place_behind_anchors(ops, is_bucket, anchor_of, is_final);
        CHECK(ops == (std::vector<std::string>{"f0", "f1", "b1", "B0@b1", "B1@b1", "b0", "B2@b0",
                                               "B3@gone", "END"}));
        // nothing to move: unchanged
        std::vector<std::string> plain = {"f0", "b0", "END"};
        b200_place_behind_anchors(plain, is_bucket, anchor_of, is_final);
        CHECK(plain == (std::vector<std::string>{"f0", "b0", "END"}));
    }
    // random programs: always well formed
    srand(7);
    for(int trial = 0; trial < 200; trial++) {
        std::vector<B200PlanEntry> f;
        const int k = 1 + rand() % 40;
        for(int i = 0; i < k; i++)
            f.push_back({rand() % 4 ? B200OPT_HALF : B200OPT_FLOAT, (size_t)(1 + rand() % 100000),
                         (long)(rand() % 30) - 1});
        for(int graph = 0; graph < 2; graph++) {
            B200Plan p = b200_plan_buckets(f, 1 + rand() % 9, graph != 0);
            if(well_formed(f, p))
                return 1;
        }
    }
    printf("ok\n");
    return 0;
}
'''


def test_bucket_planner(tmp_path, built_library):
    src = tmp_path / "plan.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "plan"
    libdir = os.path.join(ROOT, "saga_b200")
    res = subprocess.run(["g++", "-std=c++17", "-O1", str(src), "-o", str(exe),
                          "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "saga_b200", "host"),
                          "-L", libdir, "-lb200opt", "-Wl,-rpath," + libdir, "-lpthread"],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and res.stdout.strip().endswith("ok"), res.stdout + res.stderr
