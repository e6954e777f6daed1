#include "bootstrap/launcher.hpp"

#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cerrno>
#include <cstdlib>
#include <cstring>

#include "core/env.hpp"
#include "core/log.hpp"

namespace cclx {

bool pmi1_client::available() {
    return std::getenv("PMI_FD") != nullptr || std::getenv("PMI_PORT") != nullptr;
}

std::string pmi1_client::field(const std::string& line, const char* key) {
    const std::string k = std::string(key) + "=";
    size_t pos = 0;
    while ((pos = line.find(k, pos)) != std::string::npos) {
        if (pos == 0 || line[pos - 1] == ' ') {
            const size_t b = pos + k.size();
            size_t e = line.find(' ', b);
            if (e == std::string::npos)
                e = line.size();
            return line.substr(b, e - b);
        }
        pos += k.size();
    }
    return "";
}

std::string pmi1_client::read_line() {
    for (;;) {
        const size_t nl = pending_.find('\n');
        if (nl != std::string::npos) {
            std::string line = pending_.substr(0, nl);
            pending_.erase(0, nl + 1);
            return line;
        }
        char buf[2048];
        const ssize_t n = ::read(fd_, buf, sizeof(buf));
        if (n < 0 && errno == EINTR)
            continue;
        CCL_THROW_IF_NOT(n > 0, "the process manager closed the PMI connection");
        pending_.append(buf, (size_t)n);
    }
}

std::string pmi1_client::roundtrip(const std::string& line, const char* expect) {
    std::string out = line + "\n";
    size_t sent = 0;
    while (sent < out.size()) {
        const ssize_t n = ::write(fd_, out.data() + sent, out.size() - sent);
        if (n < 0 && errno == EINTR)
            continue;
        CCL_THROW_IF_NOT(n > 0, "can not write to the process manager: ", std::strerror(errno));
        sent += (size_t)n;
    }
    if (!expect)
        return "";
    const std::string answer = read_line();
    CCL_THROW_IF_NOT(field(answer, "cmd") == expect, "PMI: sent '", line, "', expected cmd=", expect, ", got '", answer,
                     "'");
    const std::string rc = field(answer, "rc");
    CCL_THROW_IF_NOT(rc.empty() || rc == "0", "PMI: '", line, "' failed: ", answer);
    return answer;
}

pmi1_client::pmi1_client() {
    if (const char* fd = std::getenv("PMI_FD")) {
        fd_ = std::atoi(fd);
        if (const char* r = std::getenv("PMI_RANK"))
            rank_ = std::atoi(r);
        if (const char* s = std::getenv("PMI_SIZE"))
            size_ = std::atoi(s);
    }
    else {
        // PMI_PORT=host:port: connect and identify with PMI_ID; the manager answers with size and rank
        const std::string hp = std::getenv("PMI_PORT");
        const size_t colon = hp.rfind(':');
        CCL_THROW_IF_NOT(colon != std::string::npos, "PMI_PORT must be host:port, got ", hp);
        addrinfo hints{}, *res = nullptr;
        hints.ai_socktype = SOCK_STREAM;
        CCL_THROW_IF_NOT(getaddrinfo(hp.substr(0, colon).c_str(), hp.substr(colon + 1).c_str(), &hints, &res) == 0 && res,
                         "can not resolve PMI_PORT ", hp);
        fd_ = ::socket(res->ai_family, res->ai_socktype | SOCK_CLOEXEC, res->ai_protocol);
        const bool ok = fd_ >= 0 && ::connect(fd_, res->ai_addr, res->ai_addrlen) == 0;
        freeaddrinfo(res);
        CCL_THROW_IF_NOT(ok, "can not connect to the process manager at ", hp, ": ", std::strerror(errno));
        own_fd_ = true;
        const char* id = std::getenv("PMI_ID");
        roundtrip(std::string("cmd=initack pmiid=") + (id ? id : "0"), "initack");
        for (int i = 0; i < 3; i++) { // cmd=set size=.. / rank=.. / debug=..
            const std::string line = read_line();
            if (!field(line, "size").empty())
                size_ = std::atoi(field(line, "size").c_str());
            if (!field(line, "rank").empty())
                rank_ = std::atoi(field(line, "rank").c_str());
        }
    }
    CCL_THROW_IF_NOT(fd_ >= 0 && rank_ >= 0 && size_ > 0, "incomplete PMI environment (PMI_FD / PMI_RANK / PMI_SIZE)");
    roundtrip("cmd=init pmi_version=1 pmi_subversion=1", "response_to_init");
    roundtrip("cmd=get_maxes", "maxes");
    kvsname_ = field(roundtrip("cmd=get_my_kvsname", "my_kvsname"), "kvsname");
    CCL_THROW_IF_NOT(!kvsname_.empty(), "the process manager named no key-value space");
}

pmi1_client::~pmi1_client() {
    try {
        finalize();
    }
    catch (...) {
    }
    if (own_fd_ && fd_ >= 0)
        ::close(fd_);
}

void pmi1_client::put(const std::string& key, const std::string& value) {
    CCL_THROW_IF_NOT(value.find(' ') == std::string::npos && value.find('\n') == std::string::npos,
                     "PMI values must not contain blanks");
    roundtrip("cmd=put kvsname=" + kvsname_ + " key=" + key + " value=" + value, "put_result");
}

std::string pmi1_client::get(const std::string& key) {
    return field(roundtrip("cmd=get kvsname=" + kvsname_ + " key=" + key, "get_result"), "value");
}

void pmi1_client::barrier() {
    roundtrip("cmd=barrier_in", "barrier_out");
}

void pmi1_client::finalize() {
    if (finalized_ || fd_ < 0)
        return;
    finalized_ = true;
    roundtrip("cmd=finalize", "finalize_ack");
}

launcher_world bootstrap_from_launcher() {
    launcher_world w;
    if (pmi1_client::available()) {
        pmi1_client pm;
        w.rank = pm.rank();
        w.size = pm.size();
        w.how = "pmi-1";
        if (w.rank == 0) {
            auto main = kvs::internal_kvs::create_main();
            pm.put("ccl_kvs_address", main->get_address().str());
            w.store = main;
        }
        pm.barrier(); // the put is visible to everybody after the barrier
        if (w.rank != 0)
            w.store = kvs::internal_kvs::create_peer(kvs::address::from_string(pm.get("ccl_kvs_address")));
        pm.barrier(); // nobody finalizes while others still read
        LOG_INFO("launcher: PMI-1, rank ", w.rank, " of ", w.size);
        return w;
    }
    const char* rank = std::getenv("RANK");
    const char* size = std::getenv("WORLD_SIZE");
    const char* addr = std::getenv("MASTER_ADDR");
    const char* port = std::getenv("MASTER_PORT");
    if (rank && size && addr && port) {
        w.rank = std::atoi(rank);
        w.size = std::atoi(size);
        w.how = "torchrun";
        std::string ip = addr;
        if (ip == "localhost")
            ip = "127.0.0.1";
        int offset = 1;
        if (const char* o = std::getenv("CCL_KVS_PORT_OFFSET"))
            offset += std::atoi(o);
        const std::string ip_port = ip + "_" + std::to_string(std::atoi(port) + offset);
        if (w.rank == 0)
            w.store = kvs::internal_kvs::create_main(ip_port);
        else
            w.store = kvs::internal_kvs::create_peer(kvs::address::from_string(ip_port));
        LOG_INFO("launcher: torchrun-style variables, rank ", w.rank, " of ", w.size, ", store at ", ip_port);
        return w;
    }
    // nobody announced a world: one process, its own store
    const env_data& env = env_data::get();
    CCL_THROW_IF_NOT(env.local_size <= 1, "no launcher found (PMI_FD / PMI_PORT, or RANK + WORLD_SIZE + MASTER_ADDR + "
                                          "MASTER_PORT) although ",
                     env.local_size, " local ranks were announced");
    w.how = "single process";
    w.store = kvs::internal_kvs::create_main();
    return w;
}

} // namespace cclx
