// -*-c++-*-
//
// Host-side shim that puts the b200opt C ABI behind Saga's optimizer op
// interface.  It is meant to be compiled INSIDE the Saga tree, included from
// src/cuda/cuda_optimizer.cpp after that file's own includes ("saga.hpp",
// "cuda_common.hpp", "cuda_tensor.hpp"), with -DHAVE_B200OPT and this
// repository's include/ directory on the include path;
// saga_b200/host/e2e/build_saga_e2e.py applies the edits that use it.
//
// What it mirrors (paths relative to the Saga project root):
//   struct Optimizer / AdamF32 / AdamMixed   src/cuda/cuda_optimizer.cpp:37-194
//       -> B200Adam: one CudaOperation that runs BOTH dtype groups in one
//          fused kernel launch (reduce-scatter + Adam + all-gather + flag sum)
//   CudaProgram::create_optimizers           src/cuda/cuda_optimizer.cpp:276-292
//       -> b200_create_optimizers(): same flat layout (16-element padding, FLOAT
//          group and HALF group), tensors re-pointed into library-owned memory
//   ncclCommInitAll                          src/cuda/cuda_common.cpp:116-127
//       -> B200Rendezvous: the per-engine meeting point where the rank threads
//          exchange their handles (one std::thread per GPU, as in Saga)
//   flag block of CudaProgram::step          src/cuda/cuda_program.cpp:282-307
//       -> B200Adam::finish_step(): stream sync + flag sums + scale policy
//
// Error convention: the C ABI returns status codes; the shim turns a non-zero
// status into std::runtime_error so that CudaProgram::runOps reports it the
// way it reports any failing op (src/cuda/cuda_program.cpp:226-231).
#pragma once

#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <functional>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "b200opt.h"

namespace saga {

// Meeting point of the rank threads of one engine.  Every rank creates its own
// handle on its own device, then joins; join() returns when all ranks have
// joined and this rank has attached every peer.  A rank whose program has
// nothing to train still joins, with a null handle, so that nobody waits for it
// in vain; the wait itself is bounded and names the ranks that did not come.
// The object serves one program after the other: when the last rank of a round
// has left, the counters and the handle table start over.
class B200Rendezvous {
public:
    explicit B200Rendezvous(int nranks, int timeout_seconds = 120)
      : m_handles(nranks, nullptr), m_present(nranks, false), m_timeout_s(timeout_seconds)
    {
    }

    void join(int rank, b200opt_t *h)
    {
        const int n = (int)m_handles.size();
        std::vector<b200opt_t *> peers;
        {
            std::unique_lock<std::mutex> lock(m_mutex);
            // a new round only starts once the previous one has been left by all
            wait_or_throw(lock, [&] { return m_leaving == 0; }, "the previous round to end");
            m_handles[rank] = h;
            m_present[rank] = true;
            m_joined++;
            m_cond.notify_all();
            try {
                wait_or_throw(lock, [&] { return m_joined >= n; }, "every rank to join");
            } catch(...) {
                // take this rank out again: a later attempt starts from a clean table
                m_handles[rank] = nullptr;
                m_present[rank] = false;
                m_joined--;
                throw;
            }
            peers = m_handles;
        }
        std::string err;
        if(h) {
            for(int q = 0; q < n && err.empty(); q++) {
                if(q == rank)
                    continue;
                if(!peers[q])
                    err = "rank " + std::to_string(q) + " has no trainable tensors but rank " +
                          std::to_string(rank) + " has";
                else if(b200opt_attach_local(h, q, peers[q]) != B200OPT_OK)
                    err = std::string("b200opt_attach_local: ") + b200opt_last_error(h);
            }
        }
        // nobody may step before every rank has wired its peers; the last rank
        // out resets the object for the next program
        std::unique_lock<std::mutex> lock(m_mutex);
        m_wired++;
        m_cond.notify_all();
        try {
            wait_or_throw(lock, [&] { return m_wired >= n; }, "every rank to wire its peers");
        } catch(...) {
            leave(n);
            throw;
        }
        leave(n);
        if(!err.empty())
            throw std::runtime_error(err);
    }

private:
    // called with the mutex held, by every rank once, on its way out of a round
    void leave(int n)
    {
        if(m_leaving == 0)
            m_leaving = n;
        if(--m_leaving == 0) {
            m_joined = m_wired = 0;
            std::fill(m_handles.begin(), m_handles.end(), nullptr);
            std::fill(m_present.begin(), m_present.end(), false);
            m_cond.notify_all();
        }
    }

    template <typename Pred>
    void wait_or_throw(std::unique_lock<std::mutex> &lock, Pred pred, const char *what)
    {
        if(m_cond.wait_for(lock, std::chrono::seconds(m_timeout_s), pred))
            return;
        std::string missing;
        for(size_t q = 0; q < m_present.size(); q++)
            if(!m_present[q])
                missing += (missing.empty() ? "" : ", ") + std::to_string(q);
        throw std::runtime_error(std::string("b200opt rendezvous: gave up waiting for ") + what +
                                 (missing.empty() ? "" : " (ranks not seen: " + missing + ")"));
    }

    std::mutex m_mutex;
    std::condition_variable m_cond;
    std::vector<b200opt_t *> m_handles;
    std::vector<bool> m_present;
    int m_timeout_s;
    int m_joined = 0;
    int m_wired = 0;
    int m_leaving = 0;
};

#ifdef HAVE_B200OPT  // the part below needs Saga's own headers

// Non-owning view of library memory, so that tensor storages can alias it the
// way they alias the reference's flat allocation
// (src/cuda/cuda_optimizer.cpp:245-249).  Needs the one-line constructor
// `CudaTensorStorageMemory(void *external, int)` that the integration adds to
// src/cuda/cuda_tensor.hpp.

struct B200Adam : public CudaOperation {
    B200Adam(CudaProgram &p, b200opt_t *handle, const CudaOpArgs &inputs,
             const CudaOpArgs &outputs)
      : CudaOperation("b200-adam")
      , m_handle(handle)
      , m_inputs(inputs)
      , m_outputs(outputs)
      , m_ctx(p.m_ctx)
    {
    }

    ~B200Adam()
    {
        if(m_on_destroy)
            m_on_destroy();  // lets the owner forget the handle first
        if(m_timed_steps)
            fprintf(stderr, "{\"b200_adam_op\": {\"rank\": %d, \"steps\": %ld, \"mean_us\": %.2f}}\n",
                    m_ctx->m_nccl_rank, m_timed_steps, 1e3 * m_timed_ms / m_timed_steps);
        if(m_ev[0]) {
            cudaEventDestroy(m_ev[0]);
            cudaEventDestroy(m_ev[1]);
        }
        b200opt_destroy(m_handle);
    }

    // AdamF32::exec + AdamMixed::exec (src/cuda/cuda_optimizer.cpp:76-113,
    // 148-186): iteration counter, bias corrections, 1/scale, reduce-scatter,
    // update, all-gather -- all inside b200opt_step.  Asynchronous.
    void exec(CudaProgram &p) override
    {
        // B200OPT_TIME_OP=1: device time of the op, one event on each side of it,
        // read in note_step_done() after the step's stream synchronise
        if(m_timing < 0) {
            const char *e = getenv("B200OPT_TIME_OP");
            m_timing = e && atoi(e) ? 1 : 0;
            if(m_timing) {
                cudaEventCreate(&m_ev[0]);
                cudaEventCreate(&m_ev[1]);
            }
        }
        if(m_timing)
            cudaEventRecord(m_ev[0], p.m_ctx->m_stream);
        const int rc = b200opt_step(m_handle, p.m_pc.learning_rate,
                                    p.m_pc.l2_lambda, p.m_mp_scaling,
                                    p.m_ctx->m_stream);
        if(rc != B200OPT_OK)
            throw std::runtime_error(std::string("b200opt_step: ") +
                                     b200opt_last_error(m_handle));
        if(m_timing) {
            cudaEventRecord(m_ev[1], p.m_ctx->m_stream);
            m_pending = true;
        }
    }

    // called once the stream has been synchronised after a step
    void note_step_done()
    {
        if(!m_pending)
            return;
        m_pending = false;
        float ms = 0;
        if(cudaEventElapsedTime(&ms, m_ev[0], m_ev[1]) == cudaSuccess) {
            m_timed_ms += ms;
            m_timed_steps++;
        }
    }

    // Replaces the flag block at the end of CudaProgram::step
    // (src/cuda/cuda_program.cpp:282-307): the cross-rank flag sum has already
    // happened inside the step kernel; this waits for the stream, reads the
    // sums and applies the reference's scale policy.
    void finish_step(CudaProgram &p)
    {
        uint32_t flags[3];
        const int rc = b200opt_flags(m_handle, p.m_ctx->m_stream, flags);
        if(rc != B200OPT_OK)
            throw std::runtime_error(std::string("b200opt_flags: ") +
                                     b200opt_last_error(m_handle));
        if(p.m_mp_enabled)
            b200opt_policy_update(&p.m_mp_scaling, flags,
                                  B200OPT_POLICY_REFERENCE, nullptr, 0);
    }

    CudaOpArgs listInputs() const override { return m_inputs; }
    CudaOpArgs listOutputs() const override { return m_outputs; }

    b200opt_t *m_handle;
    int m_timing = -1;
    bool m_pending = false;
    cudaEvent_t m_ev[2] = {nullptr, nullptr};
    double m_timed_ms = 0;
    long m_timed_steps = 0;
    std::function<void()> m_on_destroy;
    CudaOpArgs m_inputs;
    CudaOpArgs m_outputs;
    const std::shared_ptr<CudaContext> m_ctx;
};

#endif  // HAVE_B200OPT

}  // namespace saga
