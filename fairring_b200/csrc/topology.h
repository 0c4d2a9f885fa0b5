// Who is where: real hosts (by kernel boot id, as the reference does in
// fairring/machine.cc:25-126) and the two-level (machine, device) grouping the
// collectives run on.  On one NVSwitch box a "machine" is a configurable group
// of GPUs (1x8, 2x4, 4x2, ...), so the client/server hierarchy can be exercised
// without a second host.
#pragma once

#include <string>
#include <vector>

#include "kvstore.h"
#include "layout.h"

namespace fairring {

struct Deployment {
  Topo topo;                 // the grouping the kernels use
  int num_hosts = 1;         // distinct boot ids
  int ranks_per_host = 1;
  bool single_host = true;   // peer memory is only reachable on one host
  bool grouping_from_env = false;
  std::vector<int> host_of_rank;
};

std::string readBootId();

// gpus_per_machine == 0: derive the grouping from the real hosts (and the rank
// numbering from the order the hosts appear in, like the reference);
// otherwise form world/gpus_per_machine virtual machines, numbered `favorable`
// or standard.  `boot_id_override` lets tests pretend to be several hosts.
Deployment detectDeployment(KvStore& store, int rank, int world, int gpus_per_machine,
                            bool favorable, const std::string& boot_id_override = "");

}  // namespace fairring
