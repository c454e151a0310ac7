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
//       -> the flag sums come from b200opt_flags and feed the reference's own
//          policy block; or, with the loss scale kept on the device
//          (B200Adam::enable_device_scale), no host synchronise at all
//   optimizer ops appended behind backward   src/cuda/cuda_program.cpp:455
//       -> B200AdamBucket: parts of the step issued between the backward ops
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

// A contiguous piece of both flat buffers that one bucket of a step covers.
struct B200BucketRange {
    size_t half_first, half_count, float_first, float_count;
};

// One trainable tensor as the planner sees it: dtype group, element count, and
// the position (in the program's op list) of the last op that writes its
// gradient or reads its weights; -1 when no op touches it.
struct B200PlanEntry {
    int dtype;
    size_t elements;
    long last_touch;
};

struct B200Plan {
    std::vector<size_t> order[2];          // per dtype group: entry indices in layout order
    std::vector<B200BucketRange> buckets;  // consecutive, together covering both buffers
    std::vector<long> anchors;             // per bucket: op position it has to follow
};

// Plans the flat layout and the buckets of one optimizer step.  `entries` come
// in the reference's order (std::map order of CudaProgram::m_updates,
// src/cuda/cuda_common.hpp:285-291).  With graph_order the layout follows the
// order in which backward finishes with the tensors (stable), so that every
// bucket is final as early as possible; otherwise the reference's order is
// kept and a bucket waits for the latest of its members.  Buckets are cut at
// tensor boundaries into `nbuckets` pieces of about equal size; anchors never
// decrease, so the buckets can be issued in index order.
inline B200Plan
b200_plan_buckets(const std::vector<B200PlanEntry> &entries, int nbuckets, bool graph_order)
{
    B200Plan plan;
    std::vector<size_t> seq(entries.size());
    for(size_t i = 0; i < seq.size(); i++)
        seq[i] = i;
    if(graph_order)
        std::stable_sort(seq.begin(), seq.end(), [&](size_t a, size_t b) {
            return entries[a].last_touch < entries[b].last_touch;
        });
    auto padded = [](size_t n) { return (n + 15) / 16 * 16; };
    size_t total = 0;
    for(const auto &e : entries)
        total += padded(e.elements);
    nbuckets = std::max(1, nbuckets);
    size_t at[2] = {0, 0}, first[2] = {0, 0}, acc = 0;
    long anchor = 0;
    for(size_t k = 0; k < seq.size(); k++) {
        const auto &e = entries[seq[k]];
        plan.order[e.dtype].push_back(seq[k]);
        at[e.dtype] += padded(e.elements);
        acc += padded(e.elements);
        anchor = std::max(anchor, e.last_touch);
        const size_t done = plan.buckets.size();
        const bool is_last_entry = k + 1 == seq.size();
        // cut where the running size comes closest to this bucket's share of the total,
        // never inside a run of tensors that the same op finishes (they become final
        // together anyway)
        bool cut = false;
        if(!is_last_entry && (long)done < nbuckets - 1) {
            const auto &next = entries[seq[k + 1]];
            const bool reached = acc * nbuckets >= total * (done + 1);
            const bool closer = (2 * acc + padded(next.elements)) * nbuckets > 2 * total * (done + 1);
            cut = (reached || closer) && !(graph_order && next.last_touch == e.last_touch);
        }
        if(cut || is_last_entry) {
            plan.buckets.push_back({first[0], at[0] - first[0], first[1], at[1] - first[1]});
            plan.anchors.push_back(anchor);
            first[0] = at[0];
            first[1] = at[1];
        }
    }
    if(plan.buckets.empty()) {
        plan.buckets.push_back({0, 0, 0, 0});
        plan.anchors.push_back(0);
    }
    return plan;
}

// Moves the bucket ops of a program's op list behind the ops they depend on.
//   is_bucket(op)  true for the ops to move (they sit at the end of the list, in
//                  bucket order, when this is called)
//   anchor_of(op)  the op a bucket has to follow
//   is_final(op)   true for the op that closes the step: a bucket whose anchor is
//                  not in the list goes right in front of it
// Everything else keeps its order; buckets keep theirs, also when several share an
// anchor.  Generic over the op type so that it can be checked without Saga's headers.
template <typename Op, typename IsBucket, typename AnchorOf, typename IsFinal>
void
b200_place_behind_anchors(std::vector<Op> &ops, IsBucket is_bucket, AnchorOf anchor_of,
                          IsFinal is_final)
{
    std::vector<Op> buckets, rest;
    for(auto &op : ops)
        (is_bucket(op) ? buckets : rest).push_back(op);
    ops = rest;
    for(auto &b : buckets) {
        auto at = std::find(ops.begin(), ops.end(), anchor_of(b));
        if(at == ops.end()) {
            at = std::find_if(ops.begin(), ops.end(), is_final);
        } else {
            ++at;
            while(at != ops.end() && is_bucket(*at))
                ++at;
        }
        ops.insert(at, b);
    }
}

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
        if(m_timed_steps) {
            // one write per line: the rank threads end at about the same time
            char line[160];
            const int len = snprintf(line, sizeof(line),
                                     "{\"b200_adam_op\": {\"rank\": %d, \"steps\": %ld, \"mean_us\": %.2f}}\n",
                                     m_ctx->m_nccl_rank, m_timed_steps, 1e3 * m_timed_ms / m_timed_steps);
            fwrite(line, 1, (size_t)len, stderr);
        }
        if(m_device_scale && getenv("B200OPT_PRINT_SCALE_LOG"))
            print_scale_log();
        for(cudaEvent_t e : {m_ev[0], m_ev[1], m_step_ev[0], m_step_ev[1], m_fork, m_join})
            if(e)
                cudaEventDestroy(e);
        if(m_side)
            cudaStreamDestroy(m_side);
        b200opt_destroy(m_handle);
    }

    // ---- loss scale kept on the device -----------------------------------
    // The step kernel reads 1/scale from device memory and applies the policy
    // of CudaProgram::step (src/cuda/cuda_program.cpp:295-302) itself; the
    // loss-gradient kernels read the scale through p.m_b200_dscale.  The host
    // no longer needs the flags, so CudaProgram::step drops its stream
    // synchronise and paces itself one step behind the device instead.
    void enable_device_scale(CudaProgram &p)
    {
        const char *cap = getenv("B200OPT_SCALE_LOG");
        const size_t log_capacity = cap ? (size_t)atol(cap) : 0;
        int rc = b200opt_device_scale_enable(m_handle, p.m_mp_scaling, B200OPT_POLICY_REFERENCE,
                                             0, log_capacity);
        if(rc == B200OPT_OK)
            rc = b200opt_device_scale_ptr(m_handle, &p.m_b200_dscale);
        if(rc != B200OPT_OK)
            throw std::runtime_error(std::string("b200opt device scale: ") +
                                     b200opt_last_error(m_handle));
        cudaEventCreateWithFlags(&m_step_ev[0], cudaEventDisableTiming);
        cudaEventCreateWithFlags(&m_step_ev[1], cudaEventDisableTiming);
        m_device_scale = true;
        m_log_capacity = log_capacity;
    }

    // End of CudaProgram::step in device-scale mode: marks the end of this
    // step's work on the stream; nobody waits for it here.
    void step_end(CudaProgram &p)
    {
        cudaEventRecord(m_step_ev[m_steps & 1], p.m_ctx->m_stream);
        m_steps++;
    }

    // Right behind the enqueue of step t: waits for the end of step t-1, which
    // makes the host run exactly one step ahead of the device.  The batch
    // callbacks that follow in CudaProgram::step touch the double-buffered
    // tensors step t-1 used, so they must not start earlier.  Also the place
    // where a wait that ran out on the device surfaces, and where the host copy
    // of the scale (shown by the UI) is refreshed without draining the stream.
    void pace(CudaProgram &p)
    {
        if(m_steps > 0)
            cudaEventSynchronize(m_step_ev[(m_steps - 1) & 1]);
        float scale = 0;
        if(b200opt_device_scale_peek(m_handle, &scale, nullptr) != B200OPT_OK)
            throw std::runtime_error(std::string("b200opt: ") + b200opt_last_error(m_handle));
        p.m_mp_scaling = scale;
    }

    // Program::getMPS in device-scale mode: a read-back behind a stream wait.
    double read_scale(const CudaProgram &p) const
    {
        float scale = 0;
        if(b200opt_device_scale_read(m_handle, p.m_ctx->m_stream, &scale, nullptr, 0, nullptr) !=
           B200OPT_OK)
            throw std::runtime_error(std::string("b200opt_device_scale_read: ") +
                                     b200opt_last_error(m_handle));
        return scale;
    }

    void print_scale_log()
    {
        std::vector<uint32_t> log(4 * std::max<size_t>(m_log_capacity, 1));
        size_t count = 0;
        float scale = 0;
        if(b200opt_device_scale_read(m_handle, m_ctx->m_stream, &scale, log.data(), m_log_capacity,
                                     &count) != B200OPT_OK)
            return;
        fprintf(stderr, "{\"b200_scale_log\": {\"rank\": %d, \"steps\": %zu, \"flags\": [",
                m_ctx->m_nccl_rank, count);
        for(size_t i = 0; i < count; i++)
            fprintf(stderr, "%s[%u, %u, %u]", i ? ", " : "", log[4 * i], log[4 * i + 1], log[4 * i + 2]);
        fprintf(stderr, "], \"scale_bits\": [");
        for(size_t i = 0; i < count; i++)
            fprintf(stderr, "%s%u", i ? ", " : "", log[4 * i + 3]);
        fprintf(stderr, "]}}\n");
    }

    // ---- one step issued as buckets behind backward ------------------------
    // The reference appends its optimizer ops behind ALL backward ops
    // (src/cuda/cuda_program.cpp:455).  With buckets, the flat layout follows
    // the order in which backward finishes with each tensor, and bucket i is
    // issued -- on a side stream, gated by an event on the program's stream --
    // as soon as the last op that writes its gradients or reads its weights has
    // been enqueued, so that its reduction and update overlap the rest of
    // backward.  The last bucket is this op itself, at the end of the program;
    // the program's stream continues behind it.
    void enable_buckets(const std::vector<B200BucketRange> &ranges)
    {
        m_buckets = ranges;
        // B200OPT_BUCKET_GRID=<ctas>: the buckets that run beside backward take this many
        // CTAs instead of a grid that fills the GPU, and so leave room for backward's own
        // kernels; the last bucket, behind which nothing else runs, keeps the full grid
        if(const char *e = getenv("B200OPT_BUCKET_GRID"))
            m_bucket_grid = std::max(0L, atol(e));
        cudaStreamCreateWithFlags(&m_side, cudaStreamNonBlocking);
        cudaEventCreateWithFlags(&m_fork, cudaEventDisableTiming);
        cudaEventCreateWithFlags(&m_join, cudaEventDisableTiming);
    }

    void issue_bucket(CudaProgram &p, size_t i)
    {
        const bool last = i + 1 == m_buckets.size();
        int rc = B200OPT_OK;
        if(i == 0)
            rc = b200opt_step_begin(m_handle);
        if(rc == B200OPT_OK) {
            cudaEventRecord(m_fork, p.m_ctx->m_stream);
            cudaStreamWaitEvent(m_side, m_fork, 0);
            const auto &r = m_buckets[i];
            if(m_bucket_grid)
                b200opt_set_option(m_handle, B200OPT_OPT_GRID, last ? 0 : m_bucket_grid);
            rc = b200opt_step_bucket(m_handle, r.half_first, r.half_count, r.float_first,
                                     r.float_count, p.m_pc.learning_rate, p.m_pc.l2_lambda,
                                     p.m_mp_scaling, m_side, last ? 1 : 0);
        }
        if(rc != B200OPT_OK)
            throw std::runtime_error(std::string("b200opt_step_bucket: ") +
                                     b200opt_last_error(m_handle));
        if(last) {
            cudaEventRecord(m_join, m_side);
            cudaStreamWaitEvent(p.m_ctx->m_stream, m_join, 0);
        }
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
            m_timing = e && atoi(e) && !m_device_scale ? 1 : 0;
            if(m_timing) {
                cudaEventCreate(&m_ev[0]);
                cudaEventCreate(&m_ev[1]);
            }
        }
        if(m_timing)
            cudaEventRecord(m_ev[0], p.m_ctx->m_stream);
        if(!m_buckets.empty()) {
            issue_bucket(p, m_buckets.size() - 1);
        } else {
            const int rc = m_device_scale
                               ? b200opt_step_device_scale(m_handle, p.m_pc.learning_rate,
                                                           p.m_pc.l2_lambda, p.m_ctx->m_stream)
                               : b200opt_step(m_handle, p.m_pc.learning_rate, p.m_pc.l2_lambda,
                                              p.m_mp_scaling, p.m_ctx->m_stream);
            if(rc != B200OPT_OK)
                throw std::runtime_error(std::string("b200opt_step: ") +
                                         b200opt_last_error(m_handle));
        }
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

    // For a tree that prefers to drop the flag block at the end of
    // CudaProgram::step (src/cuda/cuda_program.cpp:282-307) altogether: waits
    // for the stream, reads the flag sums (formed across ranks inside the step
    // kernel) and applies the reference's scale policy.
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
    bool m_device_scale = false;
    size_t m_log_capacity = 0;
    cudaEvent_t m_step_ev[2] = {nullptr, nullptr};
    long m_steps = 0;
    std::vector<B200BucketRange> m_buckets;
    long m_bucket_grid = 0;
    cudaStream_t m_side = nullptr;
    cudaEvent_t m_fork = nullptr, m_join = nullptr;
    std::function<void()> m_on_destroy;
    CudaOpArgs m_inputs;
    CudaOpArgs m_outputs;
    const std::shared_ptr<CudaContext> m_ctx;
};

// One of the earlier buckets of a step: placed by b200_place_buckets right
// behind the op `m_after`, the last one that writes the bucket's gradients or
// reads its weights.
struct B200AdamBucket : public CudaOperation {
    B200AdamBucket(std::shared_ptr<B200Adam> whole, size_t index,
                   std::shared_ptr<CudaOperation> after, const CudaOpArgs &inputs,
                   const CudaOpArgs &outputs)
      : CudaOperation("b200-adam-bucket")
      , m_whole(whole)
      , m_index(index)
      , m_after(after)
      , m_inputs(inputs)
      , m_outputs(outputs)
    {
    }

    void exec(CudaProgram &p) override { m_whole->issue_bucket(p, m_index); }

    CudaOpArgs listInputs() const override { return m_inputs; }
    CudaOpArgs listOutputs() const override { return m_outputs; }

    const std::shared_ptr<B200Adam> m_whole;
    const size_t m_index;
    const std::shared_ptr<CudaOperation> m_after;
    CudaOpArgs m_inputs;
    CudaOpArgs m_outputs;
};

#endif  // HAVE_B200OPT

}  // namespace saga
