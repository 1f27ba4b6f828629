// Host-side model of the barrier protocol of the sm_100a GEMM kernels (no GPU involved).
//
// compute-sanitizer's race checker is not available where these kernels are developed, and the
// reference's only runtime check is a device assert (gemm/gemm_sm90.cu:15).  What can be checked
// without a GPU is the protocol itself: the shared-memory ring (full / empty barriers, stage and phase
// arithmetic), the accumulator hand-over between the MMA issuer and the epilogue warps (tmem_full /
// tmem_empty, their arrival counts and parities) and, for the 256 x 512 kernel, the skewed chunk
// schedule of the two accumulator halves.  The model runs the roles of ONE CTA group - the producers of
// its CTAs, the TMA engines that complete their loads later and out of order, the MMA issuer, the tensor
// pipe that executes issued operations later and in order, and the epilogue warps - as cooperative
// agents over modelled mbarriers.  Exactly one agent runs at a time; at every point where a role of the
// kernel waits or an asynchronous engine may act, a seeded generator picks who runs next, so a run is
// reproducible and different seeds explore different interleavings.  The roles use the same work-item
// decoding and chunk schedule as the kernels (gemm_plan.h) and the same parity expressions.
//
// Invariants checked (the return code names the first one broken):
//   1  deadlock: somebody waits and nobody can run
//   2  a load was issued into a ring stage whose previous contents had not been read by every MMA
//   3  an MMA executed on a stage that did not hold the K block it expected, or whose loads were in flight
//   4  an MMA wrote into an accumulator the epilogue had not finished reading
//   5  the epilogue read an accumulator that was not the final sum of its work item
//   6  an output part was written more or less than once
#include <condition_variable>
#include <functional>
#include <memory>
#include <mutex>
#include <stdint.h>
#include <thread>
#include <vector>

#include "../../include/spork_b200.h"
#include "gemm_plan.h"

namespace {

using spork::gemm_sm100::Params;
using spork::gemm_sm100::WorkItem;

struct Abort {};

// One agent runs at a time; the baton is handed over at wait points.
class Scheduler {
public:
    explicit Scheduler(uint64_t seed) : rng_(seed * 2862933555777941757ull + 3037000493ull) {}

    int add(std::function<void(int)> body)
    {
        const int id = (int)agents_.size();
        agents_.emplace_back(new Agent);
        agents_[id]->body = std::move(body);
        return id;
    }

    // Blocks the calling agent until `cond` holds and the scheduler picks it.  Called with the baton.
    void wait_until(int self, std::function<bool()> cond)
    {
        std::unique_lock<std::mutex> lock(mu_);
        agents_[self]->ready = std::move(cond);
        hand_over(lock);
        agents_[self]->cv.wait(lock, [&] { return current_ == self || failed_; });
        if (failed_) {
            throw Abort{};
        }
    }

    void yield(int self) { wait_until(self, [] { return true; }); }

    void fail(int code)
    {
        std::unique_lock<std::mutex> lock(mu_);
        if (!failed_) {
            failed_ = true;
            error_ = code;
        }
        wake_all();
        lock.unlock();
        throw Abort{};
    }

    int run()
    {
        std::vector<std::thread> threads;
        for (size_t i = 0; i < agents_.size(); ++i) {
            agents_[i]->ready = [] { return true; };
        }
        for (size_t i = 0; i < agents_.size(); ++i) {
            threads.emplace_back([this, i] {
                {
                    std::unique_lock<std::mutex> lock(mu_);
                    agents_[i]->cv.wait(lock, [&] { return current_ == (int)i || failed_; });
                    if (failed_) {
                        agents_[i]->done = true;
                        return;
                    }
                }
                try {
                    agents_[i]->body((int)i);
                } catch (const Abort&) {
                }
                std::unique_lock<std::mutex> lock(mu_);
                agents_[i]->done = true;
                if (!failed_) {
                    hand_over(lock);
                }
            });
        }
        {
            std::unique_lock<std::mutex> lock(mu_);
            hand_over(lock);
        }
        for (auto& t : threads) {
            t.join();
        }
        return error_;
    }

    uint64_t steps() const { return steps_; }

    uint32_t random(uint32_t n)
    {
        rng_ ^= rng_ << 13;
        rng_ ^= rng_ >> 7;
        rng_ ^= rng_ << 17;
        return (uint32_t)((rng_ >> 11) % n);
    }

private:
    struct Agent {
        std::function<void(int)> body;
        std::function<bool()> ready;
        std::condition_variable cv;
        bool done = false;
    };

    void wake_all()
    {
        for (auto& a : agents_) {
            a->cv.notify_all();
        }
    }

    // Picks the next agent among those that can run.  Called with mu_ held by the agent giving up the baton.
    void hand_over(std::unique_lock<std::mutex>&)
    {
        std::vector<int> runnable;
        bool all_done = true;
        for (size_t i = 0; i < agents_.size(); ++i) {
            if (!agents_[i]->done) {
                all_done = false;
                if (agents_[i]->ready()) {
                    runnable.push_back((int)i);
                }
            }
        }
        ++steps_;
        if (runnable.empty()) {
            current_ = -1;
            if (!all_done && !failed_) {
                failed_ = true;
                error_ = 1;  // deadlock
            }
            wake_all();
        } else {
            current_ = runnable[random((uint32_t)runnable.size())];
            agents_[current_]->cv.notify_all();
        }
    }

    std::mutex mu_;
    std::vector<std::unique_ptr<Agent>> agents_;
    int current_ = -1;
    bool failed_ = false;
    int error_ = 0;
    uint64_t rng_;
    uint64_t steps_ = 0;
};

// mbarrier: a phase completes when the pending arrivals and the transaction bytes both reach zero.
struct MBar {
    uint32_t expected = 1, pending = 1, phase = 0;
    int64_t tx = 0;
    void init(uint32_t n) { expected = pending = n; }
    void settle()
    {
        if (pending == 0 && tx == 0) {
            phase ^= 1u;
            pending = expected;
        }
    }
    void arrive()
    {
        --pending;
        settle();
    }
    void arrive_expect_tx(int64_t bytes)
    {
        tx += bytes;
        arrive();
    }
    void complete_tx(int64_t bytes)
    {
        tx -= bytes;   // may run ahead of the arrival that announces the bytes (the peer CTA's loads)
        settle();
    }
    bool passed(uint32_t parity) const { return phase != parity; }  // try_wait.parity
};

struct Stage {
    uint32_t item = ~0u, kb = ~0u;  // what it holds (or is being loaded with)
    uint32_t loads_in_flight = 0;
    uint32_t reads_left = 0;        // MMA operations that still have to read these contents
};

struct Accumulator {
    uint32_t item = ~0u;
    uint32_t next_kb = 0, last_kb = 0;  // the next K block it expects, one past the last
    uint32_t readers_left = 0;          // epilogue warps (of both CTAs) that still have to read it
};

struct TensorOp {
    enum Kind { kMma, kCommit } kind;
    uint32_t stage, item, kb, acc;
    bool first;
    std::vector<MBar*> arrive;  // commit: barriers that receive one arrival
    int acc_final;              // commit: the accumulator this commit hands to the epilogue, or -1
};

struct Model {
    Params p{};
    uint32_t groups = 1, group = 0, cg = 2, stages = 4, skew = 4;
    bool wide = false;
    int inject = 0;  // a protocol bug planted on purpose, to show that the checks notice (see the entry point)
    uint32_t epi_warps = 4;
    Scheduler* sched = nullptr;
    std::vector<MBar> full, tmem_full[2], tmem_empty;   // full, tmem_empty: the leader's; tmem_full[c]: per CTA
    std::vector<MBar> empty[2];                         // per CTA
    std::vector<Stage> ring[2];                         // per CTA
    Accumulator acc[2];
    std::vector<TensorOp> tensor_queue;                 // FIFO
    size_t tensor_head = 0;
    struct Load { uint32_t cta, stage; };
    std::vector<Load> loads;                            // in flight, complete in any order
    bool issuer_done = false, producers_done[2] = {false, false};
    std::vector<uint32_t> written;                      // [item][acc][cta][warp] store count
    uint32_t num_items = 0;
    uint64_t mma_ops = 0;

    uint32_t loads_per_stage() const { return wide ? 3u : 2u; }
    uint32_t reads_per_stage() const { return wide ? 2u : 1u; }
    int64_t stage_bytes() const { return wide ? 49152 : 32768; }

    void producer(int self, uint32_t cta)
    {
        uint32_t stage = 0, phase = 0;
        for (uint32_t item = 0; item < num_items; ++item) {
            const WorkItem w = spork::gemm_sm100::group_item(p, group, groups, item);
            for (uint32_t kb = w.kb_begin; kb < w.kb_end; ++kb) {
                MBar& e = empty[cta][stage];
                if (inject != 3) {
                    sched->wait_until(self, [&e, phase] { return e.passed(phase ^ 1u); });
                }
                Stage& st = ring[cta][stage];
                if (st.reads_left != 0 || st.loads_in_flight != 0) {
                    sched->fail(2);
                }
                st.item = item;
                st.kb = kb;
                st.loads_in_flight = loads_per_stage();
                st.reads_left = reads_per_stage();
                if (cta == 0) {
                    full[stage].arrive_expect_tx(stage_bytes() * (int64_t)cg);
                }
                for (uint32_t l = 0; l < loads_per_stage(); ++l) {
                    loads.push_back(Load{cta, stage});
                }
                if (++stage == stages) {
                    stage = 0;
                    phase ^= 1u;
                }
                sched->yield(self);
            }
        }
        producers_done[cta] = true;
    }

    // The TMA engines: any load in flight may complete next.
    void tma(int self)
    {
        for (;;) {
            sched->wait_until(self, [this] {
                return !loads.empty() || (producers_done[0] && (cg == 1 || producers_done[1]));
            });
            if (loads.empty()) {
                return;
            }
            const uint32_t i = sched->random((uint32_t)loads.size());
            const Load l = loads[i];
            loads[i] = loads.back();
            loads.pop_back();
            --ring[l.cta][l.stage].loads_in_flight;
            full[l.stage].complete_tx(stage_bytes() / loads_per_stage());
        }
    }

    void enqueue_mma(uint32_t stage, uint32_t item, uint32_t kb, uint32_t a, bool first)
    {
        tensor_queue.push_back(TensorOp{TensorOp::kMma, stage, item, kb, a, first, {}, -1});
    }

    void enqueue_commit(std::vector<MBar*> bars, int acc_final = -1)
    {
        tensor_queue.push_back(TensorOp{TensorOp::kCommit, 0, 0, 0, 0, false, std::move(bars), acc_final});
    }

    // The tensor pipe: issued operations execute later, in order.
    void tensor(int self)
    {
        for (;;) {
            sched->wait_until(self, [this] { return tensor_head < tensor_queue.size() || issuer_done; });
            if (tensor_head >= tensor_queue.size()) {
                return;
            }
            const TensorOp op = tensor_queue[tensor_head++];
            if (op.kind == TensorOp::kCommit) {
                if (op.acc_final >= 0) {
                    // from now on the epilogue warps of all CTAs read this accumulator
                    acc[op.acc_final].readers_left = epi_warps * cg;
                }
                for (MBar* b : op.arrive) {
                    b->arrive();
                }
                continue;
            }
            ++mma_ops;
            for (uint32_t c = 0; c < cg; ++c) {
                Stage& st = ring[c][op.stage];
                if (st.item != op.item || st.kb != op.kb || st.loads_in_flight != 0 || st.reads_left == 0) {
                    sched->fail(3);
                }
                --st.reads_left;
            }
            Accumulator& a = acc[op.acc];
            if (op.first) {
                if (a.readers_left != 0) {
                    sched->fail(4);
                }
                const WorkItem w = spork::gemm_sm100::group_item(p, group, groups, op.item);
                a.item = op.item;
                a.next_kb = w.kb_begin;
                a.last_kb = w.kb_end;
            }
            if (a.item != op.item || a.next_kb != op.kb) {
                sched->fail(4);
            }
            ++a.next_kb;
        }
    }

    std::vector<MBar*> both(std::vector<MBar>* per_cta, uint32_t index)
    {
        std::vector<MBar*> v;
        for (uint32_t c = 0; c < cg; ++c) {
            v.push_back(&per_cta[c][index]);
        }
        return v;
    }

    // gemm_kernel: one accumulator buffer per work item, alternating (tensor memory is double buffered)
    void issuer_narrow(int self)
    {
        uint32_t stage = 0, phase = 0;
        for (uint32_t item = 0; item < num_items; ++item) {
            const WorkItem w = spork::gemm_sm100::group_item(p, group, groups, item);
            const uint32_t buf = item & 1u, acc_phase = (item >> 1) & 1u;
            MBar& te = tmem_empty[buf];
            if (inject != 2) {
                sched->wait_until(self, [&te, acc_phase] { return te.passed(acc_phase ^ 1u); });
            }
            for (uint32_t kb = w.kb_begin; kb < w.kb_end; ++kb) {
                MBar& f = full[stage];
                sched->wait_until(self, [&f, phase] { return f.passed(phase); });
                enqueue_mma(stage, item, kb, buf, kb == w.kb_begin);
                enqueue_commit(both(empty, stage));
                if (++stage == stages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            enqueue_commit(both(tmem_full, buf), (int)buf);
            sched->yield(self);
        }
        issuer_done = true;
    }

    // gemm_wide_kernel: two accumulator halves per work item, chunked schedule
    void issuer_wide(int self)
    {
        uint32_t stage = 0, phase = 0;
        for (uint32_t item = 0; item < num_items; ++item) {
            const WorkItem w = spork::gemm_sm100::group_item(p, group, groups, item);
            const uint32_t n = w.kb_end - w.kb_begin;
            const uint32_t tile_phase = item & 1u;
            uint32_t done = 0;
            while (done < n) {
                const uint32_t g = spork::gemm_sm100::wide_chunk(n, done, skew);
                const bool first = done == 0, last = done + g == n;
                for (uint32_t h = 0; h < 2; ++h) {
                    if (first && inject != 2) {
                        MBar& te = tmem_empty[h];
                        sched->wait_until(self, [&te, tile_phase] { return te.passed(tile_phase ^ 1u); });
                    }
                    uint32_t s = stage, ph = phase;
                    for (uint32_t j = 0; j < g; ++j) {
                        if (h == 0) {
                            MBar& f = full[s];
                            sched->wait_until(self, [&f, ph] { return f.passed(ph); });
                        }
                        enqueue_mma(s, item, w.kb_begin + done + j, h, first && j == 0);
                        if (h == (inject == 1 ? 0u : 1u)) {
                            enqueue_commit(both(empty, s));
                        }
                        if (++s == stages) {
                            s = 0;
                            ph ^= 1u;
                        }
                    }
                    if (last) {
                        enqueue_commit(both(tmem_full, h), (int)h);
                    }
                    if (h == 1) {
                        stage = s;
                        phase = ph;
                    }
                    sched->yield(self);
                }
                done += g;
            }
        }
        issuer_done = true;
    }

    uint32_t& written_at(uint32_t item, uint32_t a, uint32_t cta, uint32_t warp)
    {
        return written[((item * 2 + a) * 2 + cta) * 8 + warp];
    }

    // gemm_wide_kernel: H0 into registers, release; wait for H1; H0's stores interleaved with H1's copy into
    // the registers they free; release; H1's stores
    void epilogue_wide(int self, uint32_t cta, uint32_t warp)
    {
        for (uint32_t item = 0; item < num_items; ++item) {
            const uint32_t parity = item & 1u;
            for (uint32_t h = 0; h < 2; ++h) {
                MBar& tf = tmem_full[cta][h];
                sched->wait_until(self, [&tf, parity] { return tf.passed(parity); });
                if (acc[h].item != item || acc[h].next_kb != acc[h].last_kb) {
                    sched->fail(5);
                }
                sched->yield(self);   // the copy into registers takes time (h = 1: H0's stores run meanwhile)
                if (acc[h].item != item || acc[h].next_kb != acc[h].last_kb) {
                    sched->fail(5);
                }
                if (h == 1) {
                    ++written_at(item, 0, cta, warp);
                }
                --acc[h].readers_left;
                tmem_empty[h].arrive();
            }
            sched->yield(self);
            ++written_at(item, 1, cta, warp);
        }
    }

    void epilogue(int self, uint32_t cta, uint32_t warp)
    {
        if (wide) {
            epilogue_wide(self, cta, warp);
            return;
        }
        for (uint32_t item = 0; item < num_items; ++item) {
            const uint32_t halves = wide ? 2u : 1u;
            for (uint32_t h = 0; h < halves; ++h) {
                const uint32_t a = wide ? h : (item & 1u);
                const uint32_t parity = wide ? (item & 1u) : ((item >> 1) & 1u);
                MBar& tf = tmem_full[cta][a];
                sched->wait_until(self, [&tf, parity] { return tf.passed(parity); });
                const Accumulator& ac = acc[a];
                if (ac.item != item || ac.next_kb != ac.last_kb) {
                    sched->fail(5);
                }
                sched->yield(self);   // the read of tensor memory takes time
                if (acc[a].item != item || acc[a].next_kb != acc[a].last_kb) {
                    sched->fail(5);   // it changed under the reader
                }
                --acc[a].readers_left;
                tmem_empty[a].arrive();
                sched->yield(self);   // the stores follow the release (256 x 512 kernel) or precede it
                ++written_at(item, a, cta, warp);
            }
        }
    }
};

}  // namespace

extern "C" int spork_gemm_sm100_ring_model(uint32_t M, uint32_t N, uint32_t K, int block_n, int cta_group, int split_k,
                                           int max_ctas, int sm_count, int stages, int skew, uint32_t seed,
                                           uint32_t group, int inject, uint64_t* stats)
{
    using namespace spork::gemm_sm100;
    const bool wide = block_n == 512;
    if ((block_n != 64 && block_n != 128 && block_n != 256 && !wide) || (cta_group != 1 && cta_group != 2) ||
        (wide && (cta_group != 2 || split_k < 1)) || split_k < -1 || split_k == 0 || max_ctas < 0 ||
        sm_count < cta_group || stages < 1 || stages > 8 || skew < 1 || M == 0 || N == 0 || K == 0) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    Model m;
    m.inject = inject;
    m.wide = wide;
    m.cg = (uint32_t)cta_group;
    m.stages = (uint32_t)stages;
    m.skew = (uint32_t)skew > m.stages ? m.stages : (uint32_t)skew;
    m.epi_warps = wide ? 8u : 4u;
    plan_launch(m.p, m.groups, M, N, K, 128u * m.cg, (uint32_t)block_n, m.cg, 64u, split_k == -1 ? 1u : (uint32_t)split_k,
                split_k == -1, max_ctas, sm_count);
    m.p.group_m = 8;
    if (group >= m.groups) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    m.group = group;
    m.num_items = group_item_count(m.p, group, m.groups);
    Scheduler sched(seed + 1);
    m.sched = &sched;
    m.full.resize(m.stages);
    for (uint32_t c = 0; c < 2; ++c) {
        m.empty[c].resize(m.stages);
        m.ring[c].resize(m.stages);
        m.tmem_full[c].resize(2);
    }
    m.tmem_empty.resize(2);
    for (auto& b : m.tmem_empty) {
        b.init(m.epi_warps * m.cg);
    }
    m.written.assign((size_t)m.num_items * 2 * 2 * 8, 0);

    for (uint32_t c = 0; c < m.cg; ++c) {
        sched.add([&m, c](int self) { m.producer(self, c); });
    }
    sched.add([&m](int self) { m.tma(self); });
    sched.add([&m](int self) {
        if (m.wide) {
            m.issuer_wide(self);
        } else {
            m.issuer_narrow(self);
        }
    });
    sched.add([&m](int self) { m.tensor(self); });
    for (uint32_t c = 0; c < m.cg; ++c) {
        for (uint32_t w = 0; w < m.epi_warps; ++w) {
            sched.add([&m, c, w](int self) { m.epilogue(self, c, w); });
        }
    }
    int rc = sched.run();
    if (rc == 0) {
        for (uint32_t item = 0; item < m.num_items && rc == 0; ++item) {
            for (uint32_t a = 0; a < 2 && rc == 0; ++a) {
                const bool used = m.wide || a == (item & 1u);
                for (uint32_t c = 0; c < m.cg && rc == 0; ++c) {
                    for (uint32_t w = 0; w < m.epi_warps; ++w) {
                        if (m.written_at(item, a, c, w) != (used ? 1u : 0u)) {
                            rc = 6;
                            break;
                        }
                    }
                }
            }
        }
    }
    if (stats) {
        stats[0] = m.num_items;
        stats[1] = m.mma_ops;
        stats[2] = sched.steps();
        stats[3] = m.groups;
    }
    return rc;
}
