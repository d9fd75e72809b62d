#include "thread_util.h"

#include <pthread.h>
#include <sched.h>

#include "error.h"

namespace pplx {

void pin_cpu(int cpu) {
  cpu_set_t set;
  CPU_ZERO(&set);
  if (cpu < 0 || cpu >= CPU_SETSIZE) {
    throw Error(ErrorKind::kInvalidArgument, "pin_cpu: cpu index out of range: " + std::to_string(cpu));
  }
  CPU_SET(cpu, &set);
  const int rc = pthread_setaffinity_np(pthread_self(), sizeof(set), &set);
  if (rc != 0) throw Error::from_errno("pthread_setaffinity_np(cpu " + std::to_string(cpu) + ")", rc);
}

std::vector<int> current_affinity() {
  cpu_set_t set;
  CPU_ZERO(&set);
  std::vector<int> out;
  if (pthread_getaffinity_np(pthread_self(), sizeof(set), &set) != 0) return out;
  for (int i = 0; i < CPU_SETSIZE; ++i) {
    if (CPU_ISSET(i, &set)) out.push_back(i);
  }
  return out;
}

void set_thread_name(const std::string& name) {
  pthread_setname_np(pthread_self(), name.substr(0, 15).c_str());
}

}  // namespace pplx
