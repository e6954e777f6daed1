// Rank, size and the key-value store from the process launcher alone, for programs that are started
// by a process manager and have no channel of their own to carry the store's address.
//
// Two launchers are understood:
//   * a PMI-1 process manager (Hydra's mpiexec and compatibles): the "simple PMI" wire protocol on the
//     socket the manager hands down in PMI_FD (or names in PMI_PORT), the role of the reference's
//     pmi_simple client (src/atl/util/pm/pmi_rt/pmi_simple.cpp, pmi/simple_pmi.c).  Rank 0 publishes the
//     store's address in the manager's key-value space, a PMI barrier makes it visible, the others read it.
//   * torchrun-style variables (RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT): the store listens next to
//     the rendezvous port (MASTER_PORT + 1 + CCL_KVS_PORT_OFFSET).
#pragma once
#include <memory>
#include <string>

#include "bootstrap/kvs.hpp"

namespace cclx {

// Client side of the PMI-1 wire protocol: newline-terminated "cmd=... key=value ..." lines.
class pmi1_client {
public:
    static bool available(); // PMI_FD or PMI_PORT is set
    pmi1_client(); // connects and performs the init handshake; throws when the manager does not answer
    ~pmi1_client();
    int rank() const { return rank_; }
    int size() const { return size_; }
    void put(const std::string& key, const std::string& value);
    std::string get(const std::string& key);
    void barrier();
    void finalize();

private:
    // sends one command line and returns the answer as text; `expect` is the cmd= of the answer
    std::string roundtrip(const std::string& line, const char* expect);
    std::string read_line();
    static std::string field(const std::string& line, const char* key);
    int fd_ = -1;
    bool own_fd_ = false;
    int rank_ = -1, size_ = -1;
    std::string kvsname_;
    std::string pending_; // bytes read past the last newline
    bool finalized_ = false;
};

struct launcher_world {
    int rank = 0, size = 1;
    std::shared_ptr<kvs::ikvs> store;
    std::string how; // "pmi-1", "torchrun" or "single process"
};

// Throws when no launcher is recognisable and more than one rank was announced.
launcher_world bootstrap_from_launcher();

} // namespace cclx
