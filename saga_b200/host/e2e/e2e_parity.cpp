// Parity of a whole Saga training run between the unmodified library and the
// library with the b200opt optimizer op, through Saga's public API only
// (saga.hpp): a small mixed-precision classifier -- fc, relu, fc, relu, fc,
// softmax classifier; fp16 activations and weights with fp32 master copies,
// cuBLAS only (no convolution, whose algorithm cuDNN picks by timing and which
// would make two runs differ by themselves) -- trained with fixed inputs on one
// GPU, or on SAGA_CUDA_CONTEXTS GPUs with one host thread each.
//
//   saga_parity init  <dir>                 writes the model's initial tensors
//                                           (Saga's own random init) to <dir>
//   saga_parity train <dir_in> <dir_out> <steps> [oneshot]
//                                           loads the tensors of <dir_in>, trains
//                                           <steps> batches, saves the trained
//                                           tensors to <dir_out> (Graph::saveTensors,
//                                           i.e. through host tensor access), prints
//                                           one JSON line: the loss scale after every
//                                           step (bit patterns) and the mean loss.
//                                           Step by step (one Program::run per batch,
//                                           the scale read after each) or, with
//                                           "oneshot", all batches in ONE Program::run
//                                           and only the final scale.
//   E2E_LOSS_EVERY=<k>  the per-batch callback reads the loss of every k-th batch
//                       only (0: never; default 1) -- reading a tensor waits for
//                       the program's stream
//
// Linked against both library builds (build_saga_e2e.py); the test runs "init"
// once and "train" with each and compares what they leave.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "saga.hpp"

using namespace saga;

int main(int argc, char **argv)
{
    if(argc < 3) {
        fprintf(stderr, "usage: %s init <dir> | train <dir_in> <dir_out> <steps>\n", argv[0]);
        return 2;
    }
    const bool init = !strcmp(argv[1], "init");
    const int steps = (!init && argc > 4) ? atoi(argv[4]) : 0;
    const bool oneshot = !init && argc > 5 && !strcmp(argv[5], "oneshot");
    const long loss_every = getenv("E2E_LOSS_EVERY") ? atol(getenv("E2E_LOSS_EVERY")) : 1;
    const int batch_size = 64, hw = 16, classes = 10;
    const auto dt = Tensor::DataType::HALF;

    Graph g;
    if(!init)
        g.loadTensors(argv[2]);  // found by name when the nodes below are created

    auto x = makeTensor(Tensor::DataType::U8, Dims({DimParam::BATCH_SIZE, 1, hw, hw}), "input");
    auto n = g.addConvert(x, dt, 1.0f / 255.0f);
    n = g.addNode("fc", n->y(), {{"outputs", 96}, {"bias", true}}, "fc1");
    n = g.addNode("relu", n->y());
    n = g.addNode("fc", n->y(), {{"outputs", 48}, {"bias", true}}, "fc2");
    n = g.addNode("relu", n->y());
    n = g.addNode("fc", n->y(), {{"outputs", classes}, {"bias", true}}, "fc3");
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

    auto engine = createEngine(make_nui());
    const char *ctx_env = getenv("SAGA_CUDA_CONTEXTS");
    auto contexts = engine->createContexts(ctx_env && atoi(ctx_env) > 1);
    const int ranks = (int)contexts.size();
    auto barrier = Barrier::make(ranks);
    std::vector<float> scales;  // rank 0's
    double loss_mean = 0;
    int failed = 0;

    // one host thread per context, as in Saga's own multi-GPU tests; rank r trains on
    // its own deterministic batches (one byte pattern per batch index and rank)
    auto rank_main = [&](int r) {
        auto &ctx = contexts[r];
        double loss_sum = 0;
        long loss_cnt = 0;
        auto pre_ops = [&](long batch, const Program &, auto tas) {
            std::vector<uint8_t> pixels((size_t)batch_size * hw * hw);
            uint32_t s = 1234567u + (uint32_t)batch * 7919u + (uint32_t)r * 104729u;
            for(auto &p : pixels) {
                s = s * 1664525u + 1013904223u;
                p = (uint8_t)(s >> 24);
            }
            tas[x]->copyBytesFrom({}, pixels.data(), pixels.size());
            auto &labels = *tas[LABELS];
            for(int i = 0; i < batch_size; i++)
                labels.set({i}, (int)(((uint32_t)(batch * batch_size + i + r) * 2654435761u) >> 28) % classes);
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
                               .learning_rate = 1e-3,
                               .l2_lambda = 0.01,
                               .tensor_layout = TensorLayout::NHWC};
        const ProgramSource ps{.graph = g, .batched_tensors = bt, .batch_size = batch_size};
        auto training = ctx->createProgram(ps, ProgramType::TRAINING, pc);
        training->finalize();

        if(init) {
            if(r == 0 && !g.saveTensors(argv[2], ctx.get())) {
                fprintf(stderr, "could not save the initial tensors to %s\n", argv[2]);
                failed = 1;
            }
            return;
        }
        barrier->wait();
        if(oneshot) {
            training->run(steps, nullptr, 0);
            if(r == 0)
                scales.push_back(training->getMPS());
        } else {
            for(int s = 0; s < steps; s++) {
                training->run(1, nullptr, s);
                if(r == 0)
                    scales.push_back(training->getMPS());
            }
        }
        barrier->wait();
        if(r == 0) {
            loss_mean = loss_cnt ? loss_sum / loss_cnt : 0.0;
            if(!g.saveTensors(argv[3], ctx.get())) {
                fprintf(stderr, "could not save the trained tensors to %s\n", argv[3]);
                failed = 1;
            }
        }
        barrier->wait();  // nobody tears its program down while rank 0 still reads
    };
    std::vector<std::thread> threads;
    for(int r = 0; r < ranks; r++)
        threads.emplace_back(rank_main, r);
    for(auto &th : threads)
        th.join();
    if(failed)
        return 1;
    if(init) {
        printf("{\"parity\": \"init\", \"dir\": \"%s\"}\n", argv[2]);
        return 0;
    }
    printf("\n{\"parity\": \"train\", \"ranks\": %d, \"steps\": %d, \"loss_mean\": %.6f, \"scale_bits\": [",
           ranks, steps, loss_mean);
    for(size_t i = 0; i < scales.size(); i++) {
        uint32_t bits;
        memcpy(&bits, &scales[i], 4);
        printf("%s%u", i ? ", " : "", bits);
    }
    printf("]}\n");
    return 0;
}
