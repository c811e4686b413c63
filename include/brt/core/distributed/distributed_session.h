// A Session that is one rank of several (runtime/include/brt/core/distributed/distributed_session.h:
// 44-82): it knows its rank and the communicator, and Run hands the communicator to the kernels
// through the ExecutionContext.  Every rank loads its own module (LoadConfig picks it by rank).
#pragma once

#include "brt/core/distributed/distributed_backend.h"
#include "brt/core/session/session.h"
#include <string>
#include <vector>

namespace brt {

class DistributedSession : public Session {
public:
  // host / port name the reference's socket rendezvous; they are kept for source compatibility
  // and not used: the communicator arrives ready-made through SetDistributedBackend
  DistributedSession(int rank, int nranks, const std::string &host = "", int port = 0);
  ~DistributedSession() override;

  // config[rank] is this rank's module
  common::Status LoadConfig(const std::vector<std::string> &config, std::string &ir_url);

  // borrowed: must outlive every Run
  void SetDistributedBackend(DistributedBackend *backend) { distributed_backend_ = backend; }

  int GetRank() const { return rank_; }
  int GetNRanks() const { return nranks_; }
  const std::string &GetHost() const { return host_; }
  int GetPort() const { return port_; }

protected:
  int rank_;
  int nranks_;
  std::string host_;
  int port_;
};

} // namespace brt
