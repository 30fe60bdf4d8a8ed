// File rendezvous between the processes of one tensor-parallel engine (one process per GPU).
// The reference is single-GPU and has nothing of the kind; this is the smallest host-side exchange
// the backend's tensor-parallel entry points need: rank 0 publishes the 128-byte communicator id,
// every rank publishes the 64-byte handle of its peer-exchange buffer, and a final marker file per
// rank acts as a barrier.  Files are written under a temporary name and renamed, so a reader never
// sees a partial file.  The directory must be fresh for every engine start.
#pragma once
#include <string>
#include <vector>

namespace edge_fm {

class TpRendezvous {
public:
    TpRendezvous(const std::string& dir, int rank, int world, double timeout_s = 120.0);

    // rank 0 writes `bytes`, every other rank waits for them; all ranks return the same bytes
    std::vector<char> broadcast_from_root(const std::string& name, const std::vector<char>& bytes);
    // every rank contributes `bytes`; returns the contributions of all ranks in rank order
    std::vector<std::vector<char>> all_gather(const std::string& name, const std::vector<char>& bytes);
    // returns once every rank has arrived
    void barrier(const std::string& name);

private:
    void publish(const std::string& file, const std::vector<char>& bytes) const;
    std::vector<char> await(const std::string& file) const;      // throws ConfigurationError after the timeout

    std::string dir_;
    int rank_, world_;
    double timeout_s_;
};

}  // namespace edge_fm
