// End-to-end training throughput of the CIFAR variant of ResNet-18 (3x3 stem,
// no stem pooling, stages of 64/128/256/512 channels with two basic blocks each,
// global average pool, FC to 10) on synthetic 32x32x3 inputs, through Saga's
// public API only (saga.hpp): Graph, Context::createProgram, Program::run.
// The reference's own harness (test/test_classifier.cpp) only offers the
// ImageNet-style ResNet-18 behind a 224x224 spatial transform, so this model
// is assembled here from the same building blocks (Graph::addResNet).
//
//   e2e_cifar_resnet18 <batch_per_gpu> <batches_per_epoch> <epochs>
//   ranks = SAGA_CUDA_CONTEXTS (one host thread per GPU, as in Saga's own tests)
//   E2E_LOSS_EVERY=<k>: the per-batch callback reads the loss of every k-th batch
//   only (0: never; default 1) -- reading a tensor waits for the program's stream
//
// Linked once against the unmodified reference library and once against the
// library with the b200opt optimizer op; prints one JSON line.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

#include "saga.hpp"

using namespace saga;

static double now_s()
{
    using namespace std::chrono;
    return duration<double>(steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char **argv)
{
    const int batch_size = argc > 1 ? atoi(argv[1]) : 256;
    const long batches = argc > 2 ? atol(argv[2]) : 40;
    const int epochs = argc > 3 ? atoi(argv[3]) : 3;
    const auto dt = Tensor::DataType::HALF;
    const long loss_every = getenv("E2E_LOSS_EVERY") ? atol(getenv("E2E_LOSS_EVERY")) : 1;

    Graph g;
    auto x = makeTensor(Tensor::DataType::U8, Dims({DimParam::BATCH_SIZE, 3, 32, 32}), "input");
    auto n = g.addConvert(x, dt, 1.0f / 255.0f);
    n = g.addNode("conv", n->y(),
                  {{"size", 3}, {"activations", 64}, {"stride", 1}, {"pad", 1}}, "stem-conv");
    n = g.addNode("batchnorm", n->y(), {}, "stem-bn");
    n = g.addNode("relu", n->y());
    const int widths[4] = {64, 128, 256, 512};
    for(int s = 0; s < 4; s++)
        for(int b = 0; b < 2; b++)
            n = g.addResNet(n->y(), widths[s], s > 0 && b == 0,
                            "s" + std::to_string(s + 2) + "_" + std::to_string(b));
    n = g.addNode("avgpool", n->y(), {{"global", true}});
    n = g.addNode("fc", n->y(), {{"outputs", 10}, {"bias", true}}, "fc");
    n = g.addNode("catclassifier", n->y());
    // The node declares its per-sample loss output as ONE float (src/node.cpp:336-337 of
    // the Saga tree) while the backward kernel writes one float per sample
    // (src/cuda/cuda_kernels.cu:35-65): with a batch of 256 that runs a kilobyte past the
    // allocation into whichever managed block follows it.  Declared per batch here, so
    // that both library builds run this program without that overflow.
    n->m_outputs["loss"] =
        makeTensor(Tensor::DataType::FLOAT, Dims({DimParam::BATCH_SIZE, 1}), "loss");

    const auto LABELS = n->m_outputs["y"]->grad();
    const auto LOSS = n->m_outputs["loss"];
    const BatchedTensors bt{{LOSS, Phase::POST}, {LABELS, Phase::PRE}, {x, Phase::PRE}};

    // one synthetic batch, reused every step
    std::vector<uint8_t> pixels((size_t)batch_size * 3 * 32 * 32);
    uint32_t seed = 2463534242u;
    for(auto &p : pixels) {
        seed ^= seed << 13;
        seed ^= seed >> 17;
        seed ^= seed << 5;
        p = (uint8_t)seed;
    }

    auto engine = createEngine(make_nui());
    auto contexts = engine->createContexts(true);
    const int ranks = (int)contexts.size();
    auto barrier = Barrier::make(ranks);
    std::vector<double> epoch_s(epochs, 0.0), loss_mean(ranks, 0.0), scale(ranks, 0.0);

    std::vector<std::thread> threads;
    for(int r = 0; r < ranks; r++) {
        threads.emplace_back([&, r] {
            auto &ctx = contexts[r];
            double loss_sum = 0;
            long loss_cnt = 0;
            auto pre_ops = [&](long batch, const Program &, auto tas) {
                tas[x]->copyBytesFrom({}, pixels.data(), pixels.size());
                auto &labels = *tas[LABELS];
                for(int i = 0; i < batch_size; i++)
                    labels.set({i}, (int)(((uint32_t)(batch * batch_size + i + r) * 2654435761u) >> 28) % 10);
            };
            auto post_ops = [&](long batch, const Program &, auto tas) {
                if(loss_every == 0 || batch % loss_every)
                    return;
                auto &loss = *tas[LOSS];
                for(int i = 0; i < batch_size; i++)
                    loss_sum += loss.get({i});
                loss_cnt += batch_size;
            };
            const ProgramConfig pc{.pre_ops = pre_ops,
                                   .post_ops = post_ops,
                                   .learning_rate = 3e-4,
                                   .l2_lambda = 0.01,
                                   .tensor_layout = TensorLayout::NHWC};
            const ProgramSource ps{.graph = g, .batched_tensors = bt, .batch_size = batch_size};
            auto training = ctx->createProgram(ps, ProgramType::TRAINING, pc);
            training->finalize();
            for(int e = 0; e < epochs; e++) {
                barrier->wait();
                const double t0 = now_s();
                training->run(batches, nullptr, batches * r);
                barrier->wait();
                if(r == 0)
                    epoch_s[e] = now_s() - t0;
            }
            loss_mean[r] = loss_cnt ? loss_sum / loss_cnt : 0;
            scale[r] = training->getMPS();
        });
    }
    for(auto &t : threads)
        t.join();

    double sum = 0, best = 0;
    for(int e = 1; e < epochs; e++) {
        const double ips = (double)batches * batch_size * ranks / epoch_s[e];
        sum += ips;
        best = ips > best ? ips : best;
    }
    printf("\n{\"e2e\": \"cifar-resnet18\", \"gpus\": %d, \"batch_per_gpu\": %d, \"batches_per_epoch\": %ld, "
           "\"epochs_timed\": %d, \"img_per_s_mean\": %.1f, \"img_per_s_best\": %.1f, "
           "\"loss_mean_rank0\": %.4f, \"loss_scale_rank0\": %.1f}\n",
           ranks, batch_size, batches, epochs - 1, epochs > 1 ? sum / (epochs - 1) : 0.0, best,
           loss_mean[0], scale[0]);
    return 0;
}
