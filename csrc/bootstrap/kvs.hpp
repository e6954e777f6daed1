// Key-value store used for bootstrap: a TCP server thread in the process that
// created the "main" KVS and blocking clients everywhere else.
//
// Same role and address format as the reference's internal KVS
// (src/atl/util/pm/pmi_resizable_rt/pmi_resizable/kvs/internal_kvs.cpp,
// internal_kvs_server.cpp: 256-byte address holding "<ip>_<port>", CCL_KVS_IFACE /
// CCL_KVS_PREFER_IPV6 / CCL_KVS_IP_PORT, 120 s connect timeout) with a
// different wire design: requests are length-prefixed field lists, so values
// may have any size (CUDA fabric handles, address tables), GET blocks on the
// server until the key exists, and the server offers atomic ADD and a counted
// BARRIER instead of fixed 130-byte records.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace cclx {
namespace kvs {

constexpr size_t ADDRESS_BYTES = 256;
typedef std::vector<char> bytes;

struct address {
    char data[ADDRESS_BYTES];
    std::string str() const;
    static address from_string(const std::string& ip_port);
};

enum op_t : uint32_t {
    OP_SET = 1,
    OP_GET = 2, // blocks until the key exists or the timeout passes
    OP_TRYGET = 3,
    OP_DEL = 4,
    OP_ADD = 5, // atomic add on an int64 stored as decimal text
    OP_COUNT = 6, // number of keys with a prefix
    OP_LIST = 7, // keys and values with a prefix
    OP_BARRIER = 8, // (name, participants): returns when `participants` callers arrived
    OP_PING = 9,
    OP_DEL_PREFIX = 10,
    OP_SHUTDOWN = 11
};

enum status_t : uint32_t { ST_OK = 0, ST_MISSING = 1, ST_TIMEOUT = 2, ST_ERROR = 3 };

class server {
public:
    server() = default;
    ~server();
    // ip_port: "" = choose interface (CCL_KVS_IFACE, else first non-loopback, else 127.0.0.1) and a free port
    void start(const std::string& ip_port = "");
    void stop();
    address addr() const { return addr_; }
    size_t key_count();

private:
    void accept_loop();
    void serve(int fd);
    int listen_fd_ = -1;
    address addr_{};
    std::thread accept_thread_;
    std::vector<std::thread> workers_;
    std::vector<int> client_fds_;
    std::atomic<bool> stopping_{ false };
    std::mutex mu_;
    std::condition_variable cv_;
    std::map<std::string, bytes> data_;
    struct barrier_state {
        uint64_t generation = 0;
        uint32_t arrived = 0;
    };
    std::map<std::string, barrier_state> barriers_;
};

class client {
public:
    client() = default;
    ~client();
    void connect(const address& a, int timeout_sec);
    void close();
    bool connected() const { return fd_ >= 0; }

    void set(const std::string& key, const void* val, size_t len);
    void set(const std::string& key, const std::string& val) { set(key, val.data(), val.size()); }
    // blocking get: throws on timeout
    bytes get(const std::string& key, int timeout_ms);
    bool try_get(const std::string& key, bytes& out);
    void del(const std::string& key);
    void del_prefix(const std::string& prefix);
    int64_t add(const std::string& key, int64_t delta);
    size_t count(const std::string& prefix);
    std::vector<std::pair<std::string, bytes>> list(const std::string& prefix);
    void barrier(const std::string& name, uint32_t participants, int timeout_ms);
    void ping();
    void shutdown_server();

private:
    uint32_t request(uint32_t op, const std::vector<bytes>& fields, std::vector<bytes>& reply);
    int fd_ = -1;
    std::mutex mu_;
};

// What the rest of the library sees: get/set of byte strings.  Implemented by
// the internal TCP store and by an adapter over a user-supplied store
// (reference src/atl/util/pm/pmi_resizable_rt/pmi_resizable/kvs/users_kvs.cpp).
class ikvs {
public:
    virtual ~ikvs() = default;
    virtual void set(const std::string& key, const bytes& val) = 0;
    virtual bool try_get(const std::string& key, bytes& out) = 0;
    // default: poll try_get
    virtual bytes get(const std::string& key, int timeout_ms);
    virtual address get_address() const = 0;
};

class internal_kvs : public ikvs {
public:
    // main: starts a server in this process and connects to it
    static std::shared_ptr<internal_kvs> create_main(const std::string& ip_port = "");
    static std::shared_ptr<internal_kvs> create_peer(const address& a);
    void set(const std::string& key, const bytes& val) override;
    bool try_get(const std::string& key, bytes& out) override;
    bytes get(const std::string& key, int timeout_ms) override;
    address get_address() const override { return addr_; }
    client& raw() { return cli_; }
    bool is_main() const { return srv_ != nullptr; }

private:
    std::unique_ptr<server> srv_;
    client cli_;
    address addr_{};
};

// pick the address the server binds to
std::string choose_local_ip(const std::string& iface, bool prefer_ipv6);

} // namespace kvs
} // namespace cclx
