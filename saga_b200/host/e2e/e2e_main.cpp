// End-to-end training throughput of Saga with synthetic data, through the
// reference's own classifier harness: this file only supplies the callbacks
// that saga::test_classifier (test/test_classifier.h of the Saga tree) expects
// from test/mnist.cpp / test/cifar.cpp -- a synthetic input batch, uniform
// labels, and wall-clock marks at the epoch boundaries -- and prints one JSON
// line with images per second.  It is linked once against the unmodified
// reference library and once against the reference library with the b200opt
// optimizer op (see build_saga_e2e.py).
//
//   saga_e2e [test_classifier options: -h -c -b N -m resnet-50 -U -r LR ...]
//   environment: E2E_HW (input height = width, default 32), E2E_LABELS (10),
//                E2E_TRAIN_BATCHES (per GPU and epoch, default 20),
//                E2E_EPOCHS (default 3; the first is warm-up)
#include <signal.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <cstdio>
#include <vector>

#include "saga.hpp"
#include "test/test_classifier.h"

using namespace saga;

static double now_s()
{
    using namespace std::chrono;
    return duration<double>(steady_clock::now().time_since_epoch()).count();
}

static int env_int(const char *name, int dflt)
{
    const char *e = getenv(name);
    return e ? atoi(e) : dflt;
}

int main(int argc, char **argv)
{
    const int hw = env_int("E2E_HW", 32);
    const int labels = env_int("E2E_LABELS", 10);
    const int train_batches = env_int("E2E_TRAIN_BATCHES", 20);
    const int epochs = env_int("E2E_EPOCHS", 3);

    int batch_size = 64, gpus = 0;
    for(int i = 1; i + 1 < argc; i++)
        if(!strcmp(argv[i], "-b"))
            batch_size = atoi(argv[i + 1]);
    {
        const char *e = getenv("SAGA_CUDA_CONTEXTS");
        gpus = e ? atoi(e) : env_int("E2E_GPUS", 1);
    }

    const size_t train_inputs = (size_t)train_batches * batch_size * gpus;
    const size_t test_inputs = (size_t)batch_size * gpus;  // one batch per GPU

    // one synthetic batch, reused: bytes uniform in 0..255 (the harness divides
    // by the input range; the optimizer path does not care about pixel values)
    std::vector<uint8_t> pixels((size_t)batch_size * 3 * hw * hw);
    uint32_t s = 12345;
    for(auto &p : pixels) {
        s = s * 1664525u + 1013904223u;
        p = (uint8_t)(s >> 24);
    }

    auto input = makeTensor(Tensor::DataType::U8, Dims({DimParam::BATCH_SIZE, 3, hw, hw}), "input");

    std::vector<double> train_begin, train_end;
    int bs_seen = 0;

    test_classifier(
        argc, argv, input, 255, labels, train_inputs, test_inputs,
        [&](int bs, bool test) {
            bs_seen = bs;
            if(!test) {
                if((int)train_begin.size() == epochs)
                    raise(SIGINT);  // the harness stops at its next check
                train_begin.push_back(now_s());
            } else {
                train_end.push_back(now_s());
            }
        },
        [&](TensorAccess &ta, long) {
            ta.copyBytesFrom({}, pixels.data(), pixels.size());
        },
        [&](long index) -> int {
            uint32_t h = (uint32_t)index * 2654435761u;
            return (int)((h >> 16) % (uint32_t)labels);
        });

    // images per second over the epochs after the first
    double best = 0, sum = 0;
    int cnt = 0;
    for(size_t e = 1; e < train_end.size() && e < train_begin.size(); e++) {
        const double ips = train_inputs / (train_end[e] - train_begin[e]);
        best = ips > best ? ips : best;
        sum += ips;
        cnt++;
    }
    printf("\n{\"e2e\": \"saga\", \"gpus\": %d, \"batch_per_gpu\": %d, \"train_batches_per_gpu\": %d, "
           "\"epochs_timed\": %d, \"img_per_s_mean\": %.1f, \"img_per_s_best\": %.1f}\n",
           gpus, bs_seen, train_batches, cnt, cnt ? sum / cnt : 0.0, best);
    fflush(stdout);
    return 0;
}
