// nexus-run: one launcher call per node, one child process per local rank.
//
//   nexus-run [--nproc-per-node N] [--nnodes 1] [--node-rank 0] [--master-addr 127.0.0.1]
//             [--master-port 29500] [--grace-s 30] [--max-restarts K] [--restart-nproc M] [--] PROGRAM [ARG ...]
//
// Every child gets RANK, LOCAL_RANK, WORLD_SIZE, LOCAL_WORLD_SIZE, GROUP_RANK, MASTER_ADDR, MASTER_PORT,
// NEXUS_RUN=1 and NEXUS_RESTART_COUNT.  When a child exits non-zero the others get `--grace-s` seconds to
// notice (their collectives fail or time out) before the rest of the group is terminated; a table of exit
// codes per rank is printed and the launcher returns the first failure's code.  With `--max-restarts` the
// whole group is torn down at once on a failure and started again (optionally with `--restart-nproc`
// processes) on MASTER_PORT + attempt, so that the program can resume from its last checkpoint.
// Each group runs in its own process group so that termination reaches grandchildren too.
// Parity: tools/nexus_run/main.cpp:1-24,143-275 of the reference (Windows job objects there).
#include <cerrno>
#include <chrono>
#include <csignal>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <sys/types.h>
#include <sys/wait.h>
#include <unistd.h>

namespace {

struct Options {
  int nproc = 1, nnodes = 1, node_rank = 0, master_port = 29500, max_restarts = 0, restart_nproc = 0;
  double grace_s = 30.0;
  std::string master_addr = "127.0.0.1";
  std::vector<std::string> program;
};

[[noreturn]] void usage(const char* why) {
  std::fprintf(stderr,
               "nexus-run: %s\nusage: nexus-run [--nproc-per-node N] [--nnodes 1] [--node-rank 0] [--master-addr A]\n"
               "                 [--master-port P] [--grace-s S] [--max-restarts K] [--restart-nproc M] [--] PROGRAM [ARG ...]\n",
               why);
  std::exit(2);
}

Options parse(int argc, char** argv) {
  Options o;
  int i = 1;
  auto need = [&](const char* flag) -> const char* {
    if (i + 1 >= argc) usage((std::string(flag) + " needs a value").c_str());
    return argv[++i];
  };
  for (; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "--") {
      ++i;
      break;
    }
    if (a == "--nproc-per-node") o.nproc = std::atoi(need("--nproc-per-node"));
    else if (a == "--nnodes") o.nnodes = std::atoi(need("--nnodes"));
    else if (a == "--node-rank") o.node_rank = std::atoi(need("--node-rank"));
    else if (a == "--master-addr") o.master_addr = need("--master-addr");
    else if (a == "--master-port") o.master_port = std::atoi(need("--master-port"));
    else if (a == "--grace-s") o.grace_s = std::atof(need("--grace-s"));
    else if (a == "--max-restarts") o.max_restarts = std::atoi(need("--max-restarts"));
    else if (a == "--restart-nproc") o.restart_nproc = std::atoi(need("--restart-nproc"));
    else if (a.rfind("--", 0) == 0) usage(("unknown option " + a).c_str());
    else break;
  }
  for (; i < argc; ++i) o.program.emplace_back(argv[i]);
  if (o.program.empty()) usage("no program given");
  if (o.nproc < 1 || o.nnodes < 1 || o.node_rank < 0 || o.node_rank >= o.nnodes) usage("bad process / node counts");
  return o;
}

double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct Child {
  pid_t pid = -1;
  int code = -1;  // exit code, 128 + signal, or -1 while running
};

int decode(int status) {
  if (WIFEXITED(status)) return WEXITSTATUS(status);
  if (WIFSIGNALED(status)) return 128 + WTERMSIG(status);
  return 255;
}

// Runs one attempt.  Returns 0 when every rank exited 0, else the first observed failure code.
int run_group(const Options& o, int nproc, int attempt, bool elastic) {
  const int world = nproc * o.nnodes;
  const int port = o.master_port + attempt;
  std::vector<Child> kids(static_cast<size_t>(nproc));
  for (int local = 0; local < nproc; ++local) {
    const pid_t pid = fork();
    if (pid < 0) {
      std::perror("nexus-run: fork");
      return 255;
    }
    if (pid == 0) {
      setpgid(0, 0);
      const int rank = o.node_rank * nproc + local;
      setenv("RANK", std::to_string(rank).c_str(), 1);
      setenv("LOCAL_RANK", std::to_string(local).c_str(), 1);
      setenv("WORLD_SIZE", std::to_string(world).c_str(), 1);
      setenv("LOCAL_WORLD_SIZE", std::to_string(nproc).c_str(), 1);
      setenv("GROUP_RANK", std::to_string(o.node_rank).c_str(), 1);
      setenv("MASTER_ADDR", o.master_addr.c_str(), 1);
      setenv("MASTER_PORT", std::to_string(port).c_str(), 1);
      setenv("NEXUS_RUN", "1", 1);
      setenv("NEXUS_RESTART_COUNT", std::to_string(attempt).c_str(), 1);
      std::vector<char*> args;
      for (const auto& s : o.program) args.push_back(const_cast<char*>(s.c_str()));
      args.push_back(nullptr);
      execvp(args[0], args.data());
      std::fprintf(stderr, "nexus-run: cannot start %s: %s\n", args[0], std::strerror(errno));
      _exit(127);
    }
    setpgid(pid, pid);
    kids[static_cast<size_t>(local)].pid = pid;
  }
  int first_fail = 0, running = nproc;
  double deadline = -1.0;
  while (running > 0) {
    int status = 0;
    const pid_t done = waitpid(-1, &status, WNOHANG);
    if (done > 0) {
      for (auto& k : kids)
        if (k.pid == done && k.code < 0) {
          k.code = decode(status);
          --running;
          if (k.code != 0 && first_fail == 0) {
            first_fail = k.code;
            deadline = elastic ? now_s() : now_s() + o.grace_s;  // elastic: tear the group down at once
          }
        }
      continue;
    }
    if (first_fail != 0 && now_s() >= deadline) {
      for (auto& k : kids)
        if (k.code < 0) kill(-k.pid, SIGTERM);
      const double hard = now_s() + 2.0;
      while (running > 0) {
        const pid_t d2 = waitpid(-1, &status, WNOHANG);
        if (d2 > 0) {
          for (auto& k : kids)
            if (k.pid == d2 && k.code < 0) {
              k.code = decode(status);
              --running;
            }
        } else if (now_s() > hard) {
          for (auto& k : kids)
            if (k.code < 0) kill(-k.pid, SIGKILL);
          std::this_thread::sleep_for(std::chrono::milliseconds(20));
        } else {
          std::this_thread::sleep_for(std::chrono::milliseconds(5));
        }
      }
      break;
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
  std::fprintf(stderr, "nexus-run: attempt %d exit codes:", attempt);
  for (int local = 0; local < nproc; ++local)
    std::fprintf(stderr, " [rank %d: %d]", o.node_rank * nproc + local, kids[static_cast<size_t>(local)].code);
  std::fprintf(stderr, "\n");
  return first_fail;
}

}  // namespace

int main(int argc, char** argv) {
  const Options o = parse(argc, argv);
  int nproc = o.nproc;
  for (int attempt = 0;; ++attempt) {
    const bool can_restart = attempt < o.max_restarts;
    const int rc = run_group(o, nproc, attempt, can_restart);
    if (rc == 0) return 0;
    if (!can_restart) return rc;
    if (o.restart_nproc > 0) nproc = o.restart_nproc;
    std::fprintf(stderr, "nexus-run: restarting the group with %d process(es) (restart %d of %d)\n", nproc, attempt + 1,
                 o.max_restarts);
  }
}
