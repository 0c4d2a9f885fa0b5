#include "topology.h"

#include <fstream>
#include <map>

namespace fairring {

std::string readBootId() {
  std::ifstream f("/proc/sys/kernel/random/boot_id");
  std::string s;
  if (f) std::getline(f, s);
  if (s.empty()) s = "unknown-host";
  return s;
}

Deployment detectDeployment(KvStore& store, int rank, int world, int gpus_per_machine,
                            bool favorable, const std::string& boot_id_override) {
  FR_CHECK(world >= 1 && rank >= 0 && rank < world, "bad rank ", rank, " of ", world);
  const std::string mine = boot_id_override.empty() ? readBootId() : boot_id_override;
  store.setString("rdv/" + std::to_string(rank) + "/boot_id", mine);

  Deployment dep;
  dep.host_of_rank.resize(world);
  std::map<std::string, int> host_index;  // first-seen order over ranks
  std::vector<int> count;
  for (int r = 0; r < world; ++r) {
    const std::string id = store.getString("rdv/" + std::to_string(r) + "/boot_id");
    auto it = host_index.find(id);
    if (it == host_index.end()) {
      it = host_index.emplace(id, (int)host_index.size()).first;
      count.push_back(0);
    }
    dep.host_of_rank[r] = it->second;
    ++count[it->second];
  }
  dep.num_hosts = (int)host_index.size();
  for (int c : count)
    FR_CHECK(c == count[0], "every host must run the same number of ranks (saw ", c, " and ",
             count[0], ")");
  dep.ranks_per_host = count[0];
  dep.single_host = dep.num_hosts == 1;

  int D;
  bool fav;
  if (gpus_per_machine > 0) {
    FR_CHECK(world % gpus_per_machine == 0, "FAIRRING_GPUS_PER_MACHINE=", gpus_per_machine,
             " does not divide the world size ", world);
    D = gpus_per_machine;
    fav = favorable;
    dep.grouping_from_env = true;
  } else {
    D = dep.ranks_per_host;
    const int M = dep.num_hosts;
    // Which of the two numberings do the hosts follow?
    bool is_std = true, is_fav = true;
    for (int r = 0; r < world; ++r) {
      if (dep.host_of_rank[r] != r / D) is_std = false;
      if (dep.host_of_rank[r] != r % M) is_fav = false;
    }
    FR_CHECK(is_std || is_fav,
             "ranks must be numbered machine-major (m*D+d) or device-major (d*M+m)");
    fav = !is_std;  // M == 1 satisfies both: call it standard
  }
  dep.topo = makeTopo(world, D, fav, rank);
  return dep;
}

}  // namespace fairring
