// Concurrency stress of the host runtime, meant to be built with -fsanitize=thread or
// -fsanitize=address,undefined and run by tests/test_sanitizers.py. Not part of the Python module.
//
//   ring      4 producers / 4 consumers over one MpmcRing, every item seen exactly once
//   kvstore   writers, BLPOP consumers and a TTL sweeper on one KvStore
//   rdma      two RDMA endpoints on the software fabric with a 64-entry send queue: three threads issue
//             striped writes, reads and write_with_imm while a fourth drains immediates; then send / recv pairs
//             in order; then shutdown with operations still in flight (everything must complete or fail, never hang)
//   tcp       the same one-sided mix over a TcpEndpoint pair
// Exit code 0 = all checks passed. What the reference covers with stress tests that need a NIC
// (tests/python/test_stress_concurrent.py, test_stress_imm_recv.py, test_stress_send_recv.py,
// test_shutdown_cancel.py in the reference).
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "core/ring.h"
#include "ctrl/kvstore.h"
#include "transport/rdma/rdma_endpoint.h"
#include "transport/tcp_endpoint.h"

using namespace slime;

#define CHECK(cond)                                                                                \
    do {                                                                                           \
        if (!(cond)) {                                                                             \
            fprintf(stderr, "CHECK failed at %s:%d: %s\n", __FILE__, __LINE__, #cond);             \
            exit(1);                                                                               \
        }                                                                                          \
    } while (0)

static void stress_ring()
{
    MpmcRing<uint32_t>    ring(256);
    constexpr uint32_t    per = 20000;
    std::vector<std::atomic<uint8_t>> seen(4 * per);
    for (auto& s : seen) s.store(0);
    std::atomic<uint32_t> consumed{0};
    std::vector<std::thread> ts;
    for (uint32_t p = 0; p < 4; ++p)
        ts.emplace_back([&, p] {
            for (uint32_t i = 0; i < per; ++i) ring.push_blocking(p * per + i);
        });
    for (int c = 0; c < 4; ++c)
        ts.emplace_back([&] {
            uint32_t v;
            while (consumed.load() < 4 * per) {
                if (ring.try_pop(v)) {
                    CHECK(seen[v].fetch_add(1) == 0);
                    consumed.fetch_add(1);
                }
            }
        });
    for (auto& t : ts) t.join();
    for (auto& s : seen) CHECK(s.load() == 1);
    printf("ring ok\n");
}

static void stress_kvstore()
{
    ctrl::KvStore         kv;
    std::atomic<int>      got{0};
    std::atomic<bool>     stop{false};
    std::vector<std::thread> ts;
    for (int w = 0; w < 3; ++w)
        ts.emplace_back([&, w] {
            for (int i = 0; i < 2000; ++i) {
                kv.set("k:" + std::to_string(w) + ":" + std::to_string(i % 50), std::to_string(i), i % 3 == 0 ? 5 : -1);
                kv.hset("h:" + std::to_string(w), {{"f" + std::to_string(i % 7), std::to_string(i)}});
                kv.rpush("q", {std::to_string(w * 10000 + i)});
                kv.incr("counter");
            }
        });
    for (int c = 0; c < 2; ++c)
        ts.emplace_back([&] {
            while (got.load() < 6000) {
                auto r = kv.blpop({"q"}, 50);
                if (r) got.fetch_add(1);
            }
        });
    ts.emplace_back([&] {
        while (!stop.load()) {
            kv.keys("k:*");
            kv.scan(0, "h:*", 10);
            std::this_thread::sleep_for(std::chrono::milliseconds(1));
        }
    });
    for (size_t i = 0; i < 5; ++i) ts[i].join();
    stop.store(true);
    ts[5].join();
    CHECK(got.load() == 6000);
    CHECK(kv.get("counter").value_or("") == "6000");
    printf("kvstore ok\n");
}

template<typename MakePair>
static void stress_endpoints(const char* label, MakePair make_pair, bool with_sendrecv)
{
    auto [a, b] = make_pair();
    constexpr size_t n = 4 << 20;
    std::vector<uint8_t> src(n), dst(n), back(n);
    for (size_t i = 0; i < n; ++i) src[i] = static_cast<uint8_t>(i * 7 + 1);
    a->register_memory_region("src", reinterpret_cast<uintptr_t>(src.data()), 0, n);
    a->register_memory_region("back", reinterpret_cast<uintptr_t>(back.data()), 0, n);
    b->register_memory_region("dst", reinterpret_cast<uintptr_t>(dst.data()), 0, n);
    Json ia = a->endpoint_info(), ib = b->endpoint_info();
    CHECK(a->connect(ib) == 0 && b->connect(ia) == 0);
    if (a->kind() == "tcp")
        for (auto& kv : ib["mr_info"].fields()) a->register_remote_memory_region(kv.first, kv.second);
    const int32_t hs = a->local_pool()->get_mr_handle("src"), hb = a->local_pool()->get_mr_handle("back");
    const int32_t hd = a->remote_pool()->get_remote_mr_handle("dst");
    CHECK(hs >= 0 && hb >= 0 && hd >= 0);

    constexpr int kImm = 200;
    std::atomic<int> imm_seen{0};
    std::vector<std::thread> ts;
    // thread 0: many small writes in big batches (more work requests than send-queue entries)
    ts.emplace_back([&] {
        for (int round = 0; round < 20; ++round) {
            std::vector<assign_tuple_t> batch;
            for (int i = 0; i < 300; ++i) batch.emplace_back(hs, hd, (round * 300 + i) * 256ull, (round * 300 + i) * 256ull, 256);
            CHECK(a->write(batch)->wait(20000) == SUCCESS);
        }
    });
    // thread 1: large striped writes and reads of a disjoint range
    ts.emplace_back([&] {
        for (int round = 0; round < 30; ++round) {
            CHECK(a->write({assign_tuple_t{hs, hd, 2 << 20, 2 << 20, 1 << 20}})->wait(20000) == SUCCESS);
            CHECK(a->read({assign_tuple_t{hb, hd, 2 << 20, 2 << 20, 1 << 20}})->wait(20000) == SUCCESS);
        }
    });
    // thread 2: write_with_imm with increasing immediates
    ts.emplace_back([&] {
        for (int i = 0; i < kImm; ++i)
            CHECK(a->write_with_imm({assign_tuple_t{hs, hd, (3 << 20) + i * 64ull, (3 << 20) + i * 64ull, 64}}, 1000 + i)->wait(20000) == SUCCESS);
    });
    // thread 3: the receiver drains immediates; they arrive in order
    ts.emplace_back([&] {
        for (int i = 0; i < kImm; ++i) {
            auto f = b->imm_recv();
            CHECK(f->wait(20000) == SUCCESS);
            CHECK(f->imm_data() == 1000 + i);
            imm_seen.fetch_add(1);
        }
    });
    for (auto& t : ts) t.join();
    CHECK(imm_seen.load() == kImm);
    CHECK(memcmp(dst.data(), src.data(), 20 * 300 * 256) == 0);
    CHECK(memcmp(dst.data() + (2 << 20), src.data() + (2 << 20), 1 << 20) == 0);
    CHECK(memcmp(back.data() + (2 << 20), src.data() + (2 << 20), 1 << 20) == 0);
    CHECK(memcmp(dst.data() + (3 << 20), src.data() + (3 << 20), kImm * 64) == 0);

    if (with_sendrecv) {
        // two-sided: receives and sends issued from different threads, matched in order
        constexpr int kMsgs = 100;
        std::vector<std::vector<uint8_t>> out(kMsgs), in(kMsgs);
        for (int i = 0; i < kMsgs; ++i) {
            out[i].assign(100 + i * 997, static_cast<uint8_t>(i));
            in[i].assign(out[i].size(), 0);
        }
        std::thread rx([&] {
            std::vector<std::shared_ptr<RecvFuture>> fs;
            for (int i = 0; i < kMsgs; ++i) fs.push_back(b->recv(chunk_tuple_t{reinterpret_cast<uintptr_t>(in[i].data()), 0, in[i].size()}));
            for (auto& f : fs) CHECK(f->wait(20000) == SUCCESS);
        });
        std::thread tx([&] {
            std::vector<std::shared_ptr<SendFuture>> fs;
            for (int i = 0; i < kMsgs; ++i) fs.push_back(a->send(chunk_tuple_t{reinterpret_cast<uintptr_t>(out[i].data()), 0, out[i].size()}));
            for (auto& f : fs) CHECK(f->wait(20000) == SUCCESS);
        });
        rx.join();
        tx.join();
        for (int i = 0; i < kMsgs; ++i) CHECK(in[i] == out[i]);
    }

    // shutdown with work in flight: every future resolves (success or FAILED), nothing hangs, nothing is touched afterwards
    std::vector<std::shared_ptr<ReadWriteFuture>> inflight;
    for (int i = 0; i < 50; ++i) inflight.push_back(a->write({assign_tuple_t{hs, hd, 0, 0, 1 << 20}}));
    auto pending_imm = b->imm_recv();
    a->shutdown();
    b->shutdown();
    int ok = 0, failed = 0;
    for (auto& f : inflight) {
        try {
            const int32_t s = f->wait(20000);
            CHECK(s == SUCCESS);
            ++ok;
        }
        catch (const std::exception&) {
            ++failed;
        }
    }
    CHECK(ok + failed == 50);
    CHECK(pending_imm->wait(20000) == FAILED);
    a->shutdown();  // idempotent
    printf("%s ok (in-flight at shutdown: %d completed, %d failed)\n", label, ok, failed);
}

int main(int argc, char** argv)
{
    const std::string which = argc > 1 ? argv[1] : "all";
    if (which == "all" || which == "ring") stress_ring();
    if (which == "all" || which == "kvstore") stress_kvstore();
    if (which == "all" || which == "rdma") {
        setenv("SLIME_RDMA_PROVIDER", "loopback", 1);
        stress_endpoints("rdma", [] {
            auto a = rdma::RdmaEndpoint::create("rdma_lo0", 1, "", 3);
            auto b = rdma::RdmaEndpoint::create("rdma_lo2", 1, "", 3);
            return std::make_pair(std::static_pointer_cast<Endpoint>(a), std::static_pointer_cast<Endpoint>(b));
        }, true);
    }
    if (which == "all" || which == "tcp") {
        stress_endpoints("tcp", [] {
            auto a = std::make_shared<TcpEndpoint>("127.0.0.1", 0, 1);
            auto b = std::make_shared<TcpEndpoint>("127.0.0.1", 0, 1);
            return std::make_pair(std::static_pointer_cast<Endpoint>(a), std::static_pointer_cast<Endpoint>(b));
        }, true);
    }
    printf("ALL OK\n");
    return 0;
}
