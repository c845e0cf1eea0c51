"""The command-line driver's host-side agreement before NCCL sections (no GPU needed): a per-GPU thread
that failed or left must make the others skip the collective instead of waiting in it."""
import os
import subprocess
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = textwrap.dedent(r"""
    #include <atomic>
    #include <cstdio>
    #include <thread>
    #include <vector>
    #include "rendezvous.h"

    static int run(int ndev, int failing, int leaving, int passes) {
      Rendezvous rv;
      rv.ndev = ndev;
      std::vector<int> yes(ndev, 0), no(ndev, 0);
      std::vector<std::thread> th;
      for (int d = 0; d < ndev; ++d)
        th.emplace_back([&, d] {
          for (int r = 0; r < passes; ++r) {
            if (d == leaving && r == 1) break;            // ends between two agreements
            const bool mine = !(d == failing && r == 0);  // reports a failure in the first agreement
            if (rv.agree(mine)) ++yes[d];
            else ++no[d];
          }
          rv.leave();
        });
      for (auto& t : th) t.join();
      int code = 0;
      for (int d = 0; d < ndev; ++d) code = code * 100 + yes[d] * 10 + no[d];
      return code;
    }

    int main() {
      // all healthy: every thread agrees every time
      printf("%d\n", run(3, -1, -1, 3));
      // thread 1 reports a failure the first time: nobody enters that collective, later agreements are fine
      printf("%d\n", run(3, 1, -1, 3));
      // thread 2 leaves after the first agreement: that one holds, every later one is refused, nobody hangs
      printf("%d\n", run(3, -1, 2, 3));
      // a single device always agrees with itself
      printf("%d\n", run(1, -1, -1, 2));
      return 0;
    }
""")


def test_rendezvous_never_leaves_a_thread_waiting(tmp_path):
    src = tmp_path / "rv.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "rv"
    subprocess.run(["/usr/bin/g++", "-O1", "-std=c++17", "-pthread", "-I",
                    os.path.join(ROOT, "skywalker_b200", "csrc", "cli"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60, check=True).stdout.split()
    assert out[0] == "303030"          # yes=3,no=0 for each of 3 threads
    assert out[1] == "212121"          # first agreement refused, the next two held
    assert out[2] == "121210"          # threads 0, 1: one yes then two refusals; thread 2: one yes, then gone
    assert out[3] == "20"
