// File-based exchange of the KVS address for launches without mpirun: rank 0 writes the
// 256-byte address to a file, the other ranks poll for it (same role as the reference's
// examples/include/store.hpp used by its external_launcher example).
#pragma once
#include <chrono>
#include <cstdio>
#include <fstream>
#include <stdexcept>
#include <string>
#include <thread>

#include "oneapi/ccl.hpp"

inline std::shared_ptr<ccl::kvs> bootstrap_kvs(int rank, const std::string& path) {
    if (rank == 0) {
        auto kvs = ccl::create_main_kvs();
        auto addr = kvs->get_address();
        std::string tmp = path + ".tmp";
        {
            std::ofstream f(tmp, std::ios::binary);
            f.write(addr.data(), addr.size());
        }
        std::rename(tmp.c_str(), path.c_str());
        return kvs;
    }
    ccl::kvs::address_type addr;
    for (int tries = 0;; tries++) {
        std::ifstream f(path, std::ios::binary);
        if (f && f.read(addr.data(), addr.size()))
            break;
        if (tries > 6000)
            throw std::runtime_error("kvs address file never appeared: " + path);
        std::this_thread::sleep_for(std::chrono::milliseconds(10));
    }
    return ccl::create_kvs(addr);
}
