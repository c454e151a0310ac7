"""The meeting point of the rank threads (saga_b200/host/b200_adam_op.hpp), on CPU: ranks
without trainable tensors join with a null handle, the object serves one program after
the other, and a rank that never comes makes the others give up with its number."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r'''
#include <atomic>
#include <cstdio>
#include <thread>
#include <vector>
#include "b200_adam_op.hpp"

int main()
{
    const int n = 4;
    saga::B200Rendezvous rv(n, 2);
    // three programs in a row on the same engine: every round must see all ranks
    for(int round = 0; round < 3; round++) {
        std::atomic<int> through{0};
        std::vector<std::thread> ts;
        for(int r = 0; r < n; r++)
            ts.emplace_back([&, r] {
                std::this_thread::sleep_for(std::chrono::milliseconds(10 * ((r + round) % n)));
                rv.join(r, nullptr);
                through++;
            });
        for(auto &t : ts)
            t.join();
        if(through != n) {
            printf("round %d: only %d ranks came through\n", round, (int)through);
            return 1;
        }
    }
    // rank 2 never joins: the others give up after the limit and say who is missing
    std::atomic<int> gave_up{0}, named{0};
    std::vector<std::thread> ts;
    for(int r : {0, 1, 3})
        ts.emplace_back([&, r] {
            try {
                rv.join(r, nullptr);
            } catch(const std::runtime_error &e) {
                gave_up++;
                // (ranks that gave up earlier have withdrawn and are listed too)
                const std::string what = e.what();
                const size_t at = what.find("ranks not seen: ");
                if(at != std::string::npos && what.find('2', at) != std::string::npos)
                    named++;
            }
        });
    for(auto &t : ts)
        t.join();
    if(gave_up != 3 || named != 3) {
        printf("timeout case: gave_up %d named %d\n", (int)gave_up, (int)named);
        return 1;
    }
    // and the object is usable again afterwards
    std::atomic<int> through{0};
    std::vector<std::thread> again;
    for(int r = 0; r < n; r++)
        again.emplace_back([&, r] { rv.join(r, nullptr); through++; });
    for(auto &t : again)
        t.join();
    printf(through == n ? "ok\n" : "reuse after a timeout failed\n");
    return through == n ? 0 : 1;
}
'''


def test_rendezvous_rounds_and_timeout(tmp_path, built_library):
    src = tmp_path / "rv.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "rv"
    libdir = os.path.join(ROOT, "saga_b200")
    res = subprocess.run(["g++", "-std=c++17", "-O1", str(src), "-o", str(exe),
                          "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "saga_b200", "host"),
                          "-L", libdir, "-lb200opt", "-Wl,-rpath," + libdir, "-lpthread"],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and res.stdout.strip().endswith("ok"), res.stdout + res.stderr
