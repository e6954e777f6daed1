#include "bootstrap/kvs.hpp"

#include <arpa/inet.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <cstring>

#include "core/env.hpp"
#include "core/log.hpp"

namespace cclx {
namespace kvs {

// ---- address ----------------------------------------------------------------------
std::string address::str() const {
    return std::string(data, strnlen(data, ADDRESS_BYTES));
}

address address::from_string(const std::string& s) {
    address a;
    std::memset(a.data, 0, ADDRESS_BYTES);
    CCL_THROW_IF_NOT(s.size() < ADDRESS_BYTES, "kvs address too long");
    std::memcpy(a.data, s.data(), s.size());
    return a;
}

static void split_ip_port(const std::string& s, std::string& ip, int& port) {
    size_t u = s.rfind('_');
    CCL_THROW_IF_NOT(u != std::string::npos, "kvs address '", s, "' is not <ip>_<port>");
    ip = s.substr(0, u);
    port = std::atoi(s.substr(u + 1).c_str());
}

std::string choose_local_ip(const std::string& iface, bool prefer_ipv6) {
    ifaddrs* list = nullptr;
    std::string best4, best6;
    if (getifaddrs(&list) == 0) {
        for (ifaddrs* it = list; it; it = it->ifa_next) {
            if (!it->ifa_addr || !(it->ifa_flags & IFF_UP))
                continue;
            const bool loop = (it->ifa_flags & IFF_LOOPBACK) != 0;
            if (!iface.empty()) {
                if (iface != it->ifa_name)
                    continue;
            }
            else if (loop)
                continue;
            char buf[INET6_ADDRSTRLEN];
            if (it->ifa_addr->sa_family == AF_INET && best4.empty()) {
                inet_ntop(AF_INET, &((sockaddr_in*)it->ifa_addr)->sin_addr, buf, sizeof(buf));
                best4 = buf;
            }
            else if (it->ifa_addr->sa_family == AF_INET6 && best6.empty()) {
                const in6_addr& a6 = ((sockaddr_in6*)it->ifa_addr)->sin6_addr;
                if (IN6_IS_ADDR_LINKLOCAL(&a6))
                    continue;
                inet_ntop(AF_INET6, &a6, buf, sizeof(buf));
                best6 = buf;
            }
        }
        freeifaddrs(list);
    }
    if (prefer_ipv6 && !best6.empty())
        return best6;
    if (!best4.empty())
        return best4;
    if (!best6.empty())
        return best6;
    CCL_THROW_IF_NOT(iface.empty(), "interface ", iface, " has no usable address");
    return "127.0.0.1";
}

// ---- framing ----------------------------------------------------------------------
namespace {

bool read_all(int fd, void* buf, size_t n) {
    char* p = (char*)buf;
    while (n) {
        ssize_t r = ::recv(fd, p, n, 0);
        if (r == 0)
            return false;
        if (r < 0) {
            if (errno == EINTR)
                continue;
            return false;
        }
        p += r;
        n -= (size_t)r;
    }
    return true;
}

bool write_all(int fd, const void* buf, size_t n) {
    const char* p = (const char*)buf;
    while (n) {
        ssize_t r = ::send(fd, p, n, MSG_NOSIGNAL);
        if (r < 0) {
            if (errno == EINTR)
                continue;
            return false;
        }
        p += r;
        n -= (size_t)r;
    }
    return true;
}

bool send_msg(int fd, uint32_t head, const std::vector<bytes>& fields) {
    std::vector<char> out;
    auto put32 = [&](uint32_t v) {
        char b[4];
        std::memcpy(b, &v, 4);
        out.insert(out.end(), b, b + 4);
    };
    put32(head);
    put32((uint32_t)fields.size());
    for (auto& f : fields) {
        put32((uint32_t)f.size());
        out.insert(out.end(), f.begin(), f.end());
    }
    return write_all(fd, out.data(), out.size());
}

bool recv_msg(int fd, uint32_t& head, std::vector<bytes>& fields) {
    uint32_t hdr[2];
    if (!read_all(fd, hdr, 8))
        return false;
    head = hdr[0];
    if (hdr[1] > 1u << 20)
        return false;
    fields.resize(hdr[1]);
    for (auto& f : fields) {
        uint32_t len;
        if (!read_all(fd, &len, 4))
            return false;
        if (len > 1u << 30)
            return false;
        f.resize(len);
        if (len && !read_all(fd, f.data(), len))
            return false;
    }
    return true;
}

bytes to_bytes(const std::string& s) {
    return bytes(s.begin(), s.end());
}
std::string to_str(const bytes& b) {
    return std::string(b.begin(), b.end());
}
bytes u64_bytes(uint64_t v) {
    bytes b(8);
    std::memcpy(b.data(), &v, 8);
    return b;
}
uint64_t bytes_u64(const bytes& b) {
    uint64_t v = 0;
    if (b.size() >= 8)
        std::memcpy(&v, b.data(), 8);
    return v;
}

} // namespace

// ---- server -----------------------------------------------------------------------
server::~server() {
    stop();
}

void server::start(const std::string& ip_port_in) {
    const env_data& env = env_data::get();
    std::string ip;
    int port = 0;
    std::string want = ip_port_in.empty() ? env.kvs_ip_port : ip_port_in;
    // CCL_KVS_IP_EXCHANGE=env: the address is agreed outside the program, so it must be given
    CCL_THROW_IF_NOT(!want.empty() || env.kvs_ip_exchange != "env",
                     "CCL_KVS_IP_EXCHANGE=env needs the address of the main key-value store in CCL_KVS_IP_PORT");
    if (!want.empty())
        split_ip_port(want, ip, port);
    else
        ip = choose_local_ip(env.kvs_iface, env.kvs_prefer_ipv6);
    const bool v6 = ip.find(':') != std::string::npos;
    listen_fd_ = ::socket(v6 ? AF_INET6 : AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    CCL_THROW_IF_NOT(listen_fd_ >= 0, "socket failed: ", std::strerror(errno));
    int one = 1;
    setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    int rc;
    if (v6) {
        sockaddr_in6 a{};
        a.sin6_family = AF_INET6;
        a.sin6_port = htons((uint16_t)port);
        CCL_THROW_IF_NOT(inet_pton(AF_INET6, ip.c_str(), &a.sin6_addr) == 1, "bad IPv6 address ", ip);
        rc = ::bind(listen_fd_, (sockaddr*)&a, sizeof(a));
    }
    else {
        sockaddr_in a{};
        a.sin_family = AF_INET;
        a.sin_port = htons((uint16_t)port);
        CCL_THROW_IF_NOT(inet_pton(AF_INET, ip.c_str(), &a.sin_addr) == 1, "bad IPv4 address ", ip);
        rc = ::bind(listen_fd_, (sockaddr*)&a, sizeof(a));
    }
    CCL_THROW_IF_NOT(rc == 0, "kvs server can not bind ", ip, ":", port, ": ", std::strerror(errno));
    CCL_THROW_IF_NOT(::listen(listen_fd_, 1024) == 0, "listen failed: ", std::strerror(errno));
    sockaddr_storage ss;
    socklen_t sl = sizeof(ss);
    getsockname(listen_fd_, (sockaddr*)&ss, &sl);
    port = ntohs(v6 ? ((sockaddr_in6*)&ss)->sin6_port : ((sockaddr_in*)&ss)->sin_port);
    addr_ = address::from_string(ip + "_" + std::to_string(port));
    stopping_ = false;
    accept_thread_ = std::thread([this] { accept_loop(); });
    LOG_DEBUG("kvs server listening on ", addr_.str());
}

void server::stop() {
    if (listen_fd_ < 0)
        return;
    stopping_ = true;
    ::shutdown(listen_fd_, SHUT_RDWR); // wakes the accept loop; the descriptor stays valid until it has left
    if (accept_thread_.joinable())
        accept_thread_.join();
    ::close(listen_fd_);
    listen_fd_ = -1;
    {
        std::lock_guard<std::mutex> lk(mu_);
        for (int fd : client_fds_)
            ::shutdown(fd, SHUT_RDWR);
    }
    cv_.notify_all();
    for (auto& t : workers_)
        if (t.joinable())
            t.join();
    workers_.clear();
    for (int fd : client_fds_)
        ::close(fd);
    client_fds_.clear();
}

size_t server::key_count() {
    std::lock_guard<std::mutex> lk(mu_);
    return data_.size();
}

void server::accept_loop() {
    while (!stopping_) {
        int fd = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
        if (fd < 0) {
            if (stopping_)
                break;
            if (errno == EINTR || errno == ECONNABORTED)
                continue;
            break;
        }
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        std::lock_guard<std::mutex> lk(mu_);
        client_fds_.push_back(fd);
        workers_.emplace_back([this, fd] { serve(fd); });
    }
}

void server::serve(int fd) {
    uint32_t op;
    std::vector<bytes> f;
    while (!stopping_ && recv_msg(fd, op, f)) {
        std::vector<bytes> reply;
        uint32_t st = ST_OK;
        switch (op) {
            case OP_SET: {
                if (f.size() != 2) {
                    st = ST_ERROR;
                    break;
                }
                {
                    std::lock_guard<std::mutex> lk(mu_);
                    data_[to_str(f[0])] = f[1];
                }
                cv_.notify_all();
                break;
            }
            case OP_GET: {
                if (f.size() != 2) {
                    st = ST_ERROR;
                    break;
                }
                const std::string key = to_str(f[0]);
                const uint64_t ms = bytes_u64(f[1]);
                std::unique_lock<std::mutex> lk(mu_);
                bool ok = cv_.wait_for(lk, std::chrono::milliseconds(ms),
                                       [&] { return stopping_.load() || data_.count(key) != 0; });
                if (ok && data_.count(key))
                    reply.push_back(data_[key]);
                else
                    st = ST_TIMEOUT;
                break;
            }
            case OP_TRYGET: {
                std::lock_guard<std::mutex> lk(mu_);
                auto it = f.size() == 1 ? data_.find(to_str(f[0])) : data_.end();
                if (it == data_.end())
                    st = ST_MISSING;
                else
                    reply.push_back(it->second);
                break;
            }
            case OP_DEL: {
                std::lock_guard<std::mutex> lk(mu_);
                if (f.size() == 1)
                    data_.erase(to_str(f[0]));
                break;
            }
            case OP_DEL_PREFIX: {
                std::lock_guard<std::mutex> lk(mu_);
                if (f.size() == 1) {
                    const std::string p = to_str(f[0]);
                    for (auto it = data_.lower_bound(p); it != data_.end() && it->first.compare(0, p.size(), p) == 0;)
                        it = data_.erase(it);
                }
                break;
            }
            case OP_ADD: {
                if (f.size() != 2) {
                    st = ST_ERROR;
                    break;
                }
                int64_t nv;
                {
                    std::lock_guard<std::mutex> lk(mu_);
                    bytes& cur = data_[to_str(f[0])];
                    int64_t v = cur.empty() ? 0 : std::atoll(to_str(cur).c_str());
                    nv = v + (int64_t)bytes_u64(f[1]);
                    cur = to_bytes(std::to_string(nv));
                }
                cv_.notify_all();
                reply.push_back(u64_bytes((uint64_t)nv));
                break;
            }
            case OP_COUNT: {
                std::lock_guard<std::mutex> lk(mu_);
                const std::string p = f.size() == 1 ? to_str(f[0]) : std::string();
                uint64_t n = 0;
                for (auto it = data_.lower_bound(p); it != data_.end() && it->first.compare(0, p.size(), p) == 0; ++it)
                    n++;
                reply.push_back(u64_bytes(n));
                break;
            }
            case OP_LIST: {
                std::lock_guard<std::mutex> lk(mu_);
                const std::string p = f.size() == 1 ? to_str(f[0]) : std::string();
                for (auto it = data_.lower_bound(p); it != data_.end() && it->first.compare(0, p.size(), p) == 0;
                     ++it) {
                    reply.push_back(to_bytes(it->first));
                    reply.push_back(it->second);
                }
                break;
            }
            case OP_BARRIER: {
                if (f.size() != 3) {
                    st = ST_ERROR;
                    break;
                }
                const std::string name = to_str(f[0]);
                const uint32_t n = (uint32_t)bytes_u64(f[1]);
                const uint64_t ms = bytes_u64(f[2]);
                std::unique_lock<std::mutex> lk(mu_);
                barrier_state& b = barriers_[name];
                const uint64_t gen = b.generation;
                if (++b.arrived >= n) {
                    b.arrived = 0;
                    b.generation++;
                    lk.unlock();
                    cv_.notify_all();
                }
                else {
                    bool ok = cv_.wait_for(lk, std::chrono::milliseconds(ms), [&] {
                        return stopping_.load() || barriers_[name].generation != gen;
                    });
                    if (!ok || barriers_[name].generation == gen) {
                        // withdraw so that a later attempt starts clean
                        if (barriers_[name].generation == gen && barriers_[name].arrived > 0)
                            barriers_[name].arrived--;
                        st = ST_TIMEOUT;
                    }
                }
                break;
            }
            case OP_PING: break;
            case OP_SHUTDOWN: break;
            default: st = ST_ERROR;
        }
        if (!send_msg(fd, st, reply))
            break;
    }
}

// ---- client -----------------------------------------------------------------------
client::~client() {
    close();
}

void client::close() {
    if (fd_ >= 0) {
        ::shutdown(fd_, SHUT_RDWR);
        ::close(fd_);
        fd_ = -1;
    }
}

void client::connect(const address& a, int timeout_sec) {
    std::string ip;
    int port;
    split_ip_port(a.str(), ip, port);
    const bool v6 = ip.find(':') != std::string::npos;
    auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        int fd = ::socket(v6 ? AF_INET6 : AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
        CCL_THROW_IF_NOT(fd >= 0, "socket failed: ", std::strerror(errno));
        int rc;
        if (v6) {
            sockaddr_in6 s{};
            s.sin6_family = AF_INET6;
            s.sin6_port = htons((uint16_t)port);
            inet_pton(AF_INET6, ip.c_str(), &s.sin6_addr);
            rc = ::connect(fd, (sockaddr*)&s, sizeof(s));
        }
        else {
            sockaddr_in s{};
            s.sin_family = AF_INET;
            s.sin_port = htons((uint16_t)port);
            CCL_THROW_IF_NOT(inet_pton(AF_INET, ip.c_str(), &s.sin_addr) == 1, "bad kvs address ", a.str());
            rc = ::connect(fd, (sockaddr*)&s, sizeof(s));
        }
        if (rc == 0) {
            int one = 1;
            setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
            fd_ = fd;
            return;
        }
        ::close(fd);
        auto dt = std::chrono::steady_clock::now() - t0;
        CCL_THROW_IF_NOT(dt < std::chrono::seconds(timeout_sec), "can not connect to kvs server ", a.str(), " within ",
                         timeout_sec, " s: ", std::strerror(errno));
        usleep(20000);
    }
}

uint32_t client::request(uint32_t op, const std::vector<bytes>& fields, std::vector<bytes>& reply) {
    std::lock_guard<std::mutex> lk(mu_);
    CCL_THROW_IF_NOT(fd_ >= 0, "kvs client is not connected");
    CCL_THROW_IF_NOT(send_msg(fd_, op, fields), "kvs server connection lost (send)");
    uint32_t st;
    CCL_THROW_IF_NOT(recv_msg(fd_, st, reply), "kvs server connection lost (recv)");
    return st;
}

void client::set(const std::string& key, const void* val, size_t len) {
    std::vector<bytes> r;
    uint32_t st = request(OP_SET, { to_bytes(key), bytes((const char*)val, (const char*)val + len) }, r);
    CCL_THROW_IF_NOT(st == ST_OK, "kvs set failed for ", key);
}

bytes client::get(const std::string& key, int timeout_ms) {
    std::vector<bytes> r;
    uint32_t st = request(OP_GET, { to_bytes(key), u64_bytes((uint64_t)timeout_ms) }, r);
    CCL_THROW_IF_NOT(st == ST_OK && r.size() == 1, "kvs get timed out for key '", key, "' after ", timeout_ms, " ms");
    return r[0];
}

bool client::try_get(const std::string& key, bytes& out) {
    std::vector<bytes> r;
    uint32_t st = request(OP_TRYGET, { to_bytes(key) }, r);
    if (st != ST_OK || r.size() != 1)
        return false;
    out = r[0];
    return true;
}

void client::del(const std::string& key) {
    std::vector<bytes> r;
    request(OP_DEL, { to_bytes(key) }, r);
}

void client::del_prefix(const std::string& prefix) {
    std::vector<bytes> r;
    request(OP_DEL_PREFIX, { to_bytes(prefix) }, r);
}

int64_t client::add(const std::string& key, int64_t delta) {
    std::vector<bytes> r;
    uint32_t st = request(OP_ADD, { to_bytes(key), u64_bytes((uint64_t)delta) }, r);
    CCL_THROW_IF_NOT(st == ST_OK && r.size() == 1, "kvs add failed for ", key);
    return (int64_t)bytes_u64(r[0]);
}

size_t client::count(const std::string& prefix) {
    std::vector<bytes> r;
    uint32_t st = request(OP_COUNT, { to_bytes(prefix) }, r);
    CCL_THROW_IF_NOT(st == ST_OK && r.size() == 1, "kvs count failed");
    return (size_t)bytes_u64(r[0]);
}

std::vector<std::pair<std::string, bytes>> client::list(const std::string& prefix) {
    std::vector<bytes> r;
    uint32_t st = request(OP_LIST, { to_bytes(prefix) }, r);
    CCL_THROW_IF_NOT(st == ST_OK && r.size() % 2 == 0, "kvs list failed");
    std::vector<std::pair<std::string, bytes>> out;
    for (size_t i = 0; i < r.size(); i += 2)
        out.emplace_back(to_str(r[i]), r[i + 1]);
    return out;
}

void client::barrier(const std::string& name, uint32_t participants, int timeout_ms) {
    std::vector<bytes> r;
    uint32_t st = request(OP_BARRIER, { to_bytes(name), u64_bytes(participants), u64_bytes((uint64_t)timeout_ms) }, r);
    CCL_THROW_IF_NOT(st == ST_OK, "kvs barrier '", name, "' timed out after ", timeout_ms, " ms (", participants,
                     " participants expected)");
}

void client::ping() {
    std::vector<bytes> r;
    request(OP_PING, {}, r);
}

void client::shutdown_server() {
    std::vector<bytes> r;
    request(OP_SHUTDOWN, {}, r);
}

// ---- ikvs -------------------------------------------------------------------------
bytes ikvs::get(const std::string& key, int timeout_ms) {
    auto t0 = std::chrono::steady_clock::now();
    bytes out;
    useconds_t nap = 200;
    while (!try_get(key, out)) {
        auto dt = std::chrono::steady_clock::now() - t0;
        CCL_THROW_IF_NOT(dt < std::chrono::milliseconds(timeout_ms), "kvs get timed out for key '", key, "'");
        usleep(nap);
        if (nap < 20000)
            nap *= 2;
    }
    return out;
}

std::shared_ptr<internal_kvs> internal_kvs::create_main(const std::string& ip_port) {
    auto k = std::make_shared<internal_kvs>();
    k->srv_.reset(new server());
    k->srv_->start(ip_port);
    k->addr_ = k->srv_->addr();
    k->cli_.connect(k->addr_, env_data::get().kvs_connection_timeout_sec);
    return k;
}

std::shared_ptr<internal_kvs> internal_kvs::create_peer(const address& a) {
    auto k = std::make_shared<internal_kvs>();
    k->addr_ = a;
    k->cli_.connect(a, env_data::get().kvs_connection_timeout_sec);
    return k;
}

void internal_kvs::set(const std::string& key, const bytes& val) {
    cli_.set(key, val.data(), val.size());
}
bool internal_kvs::try_get(const std::string& key, bytes& out) {
    return cli_.try_get(key, out);
}
bytes internal_kvs::get(const std::string& key, int timeout_ms) {
    return cli_.get(key, timeout_ms);
}

} // namespace kvs
} // namespace cclx
