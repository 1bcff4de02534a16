// mccl-agent: stand-alone node agent (answers the cluster manager's pings,
// keeps region / kernel tables, reports counters).  Usage: mccl-agent [port] [--any]
#include <csignal>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unistd.h>

#include "../cluster/agent.hpp"

int main(int argc, char** argv) {
  std::signal(SIGPIPE, SIG_IGN);
  int port = 29700;
  bool any = false;
  for (int i = 1; i < argc; ++i) {
    if (std::strcmp(argv[i], "--any") == 0) any = true;
    else port = std::atoi(argv[i]);
  }
  mccl::AgentServer agent;
  try {
    int bound = agent.start(port, any);
    std::printf("mccl-agent listening on port %d\n", bound);
    std::fflush(stdout);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "mccl-agent: %s\n", e.what());
    return 1;
  }
  while (agent.running()) ::usleep(100000);
  agent.stop();
  return 0;
}
