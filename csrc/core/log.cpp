#include "core/log.hpp"

#include <chrono>
#include <cstring>
#include <ctime>
#include <unistd.h>

namespace cclx {

static const char* level_names[] = { "ERROR", "WARN", "INFO", "DEBUG", "TRACE" };

logger::logger() {
    if (const char* lv = std::getenv("CCL_LOG_LEVEL"))
        set_level(lv);
    if (const char* a = std::getenv("CCL_ABORT_ON_THROW"))
        abort_on_throw_ = std::atoi(a) != 0;
    if (const char* f = std::getenv("CCL_LOG_FILE")) {
        std::string path = std::string(f) + "." + std::to_string((long)getpid());
        if (FILE* fp = std::fopen(path.c_str(), "w"))
            sink_ = fp;
    }
}

logger& logger::get() {
    static logger inst;
    return inst;
}

bool logger::set_level(const std::string& name) {
    static const char* names[] = { "error", "warn", "info", "debug", "trace" };
    for (int i = 0; i < 5; i++) {
        if (name == names[i] || name == std::to_string(i)) {
            level_ = (log_level)i;
            return true;
        }
    }
    return false;
}

void logger::write(log_level l, const char* file, int line, const char* func, const std::string& msg) {
    using namespace std::chrono;
    auto now = system_clock::now();
    std::time_t t = system_clock::to_time_t(now);
    long us = (long)(duration_cast<microseconds>(now.time_since_epoch()).count() % 1000000);
    struct tm tmv;
    localtime_r(&t, &tmv);
    char ts[32];
    std::strftime(ts, sizeof(ts), "%H:%M:%S", &tmv);
    const char* base = std::strrchr(file, '/');
    base = base ? base + 1 : file;
    std::lock_guard<std::mutex> lk(mu_);
    if ((int)l >= (int)log_level::debug || l == log_level::error)
        std::fprintf(sink_, "%s.%06ld |CCL_%s|%s%s %s:%d %s: %s\n", ts, us, level_names[(int)l],
                     rank_ >= 0 ? " r" : "", rank_ >= 0 ? std::to_string(rank_).c_str() : "", base,
                     line, func, msg.c_str());
    else
        std::fprintf(sink_, "%s.%06ld |CCL_%s|%s%s %s\n", ts, us, level_names[(int)l],
                     rank_ >= 0 ? " r" : "", rank_ >= 0 ? std::to_string(rank_).c_str() : "",
                     msg.c_str());
    std::fflush(sink_);
}

void throw_error(const char* file, int line, const char* func, const std::string& msg) {
    const char* base = std::strrchr(file, '/');
    base = base ? base + 1 : file;
    std::string full = strcat_all(base, ":", line, " ", func, ": EXCEPTION: ", msg);
    if (logger::get().abort_on_throw()) {
        LOG_ERROR(full);
        std::abort();
    }
    throw exception(full);
}

} // namespace cclx
