// Leveled logger and throw/assert macros.
//
// Behavioural counterpart of the reference logger (src/common/log/log.hpp:33-421):
// five levels selected by CCL_LOG_LEVEL, a "file:line func:" prefix on
// debug/trace records, CCL_THROW / CCL_THROW_IF_NOT building a ccl::exception,
// and CCL_ABORT_ON_THROW turning every throw into abort() for core dumps.
// The design here is a single mutex-protected sink writing whole records to
// stderr (or CCL_LOG_FILE), formatted with a variadic stream fold instead of
// a persistent streambuf.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>

namespace cclx {

enum class log_level : int { error = 0, warn = 1, info = 2, debug = 3, trace = 4 };

class exception : public std::runtime_error {
public:
    explicit exception(const std::string& what) : std::runtime_error(what) {}
};

class logger {
public:
    static logger& get();
    log_level level() const { return level_; }
    void set_level(log_level l) { level_ = l; }
    bool set_level(const std::string& name);
    bool abort_on_throw() const { return abort_on_throw_; }
    void set_abort_on_throw(bool v) { abort_on_throw_ = v; }
    void set_rank(int r) { rank_ = r; }
    void write(log_level l, const char* file, int line, const char* func, const std::string& msg);

private:
    logger();
    log_level level_ = log_level::warn;
    bool abort_on_throw_ = false;
    int rank_ = -1;
    FILE* sink_ = stderr;
    std::mutex mu_;
};

template <class... Args>
inline std::string strcat_all(Args&&... args) {
    std::ostringstream ss;
    (void)std::initializer_list<int>{ ((ss << args), 0)... };
    return ss.str();
}

[[noreturn]] void throw_error(const char* file, int line, const char* func, const std::string& msg);

} // namespace cclx

#define CCLX_LOG(lvl, ...) \
    do { \
        if ((int)(lvl) <= (int)::cclx::logger::get().level()) \
            ::cclx::logger::get().write((lvl), __FILE__, __LINE__, __func__, \
                                        ::cclx::strcat_all(__VA_ARGS__)); \
    } while (0)

#define LOG_ERROR(...) CCLX_LOG(::cclx::log_level::error, __VA_ARGS__)
#define LOG_WARN(...) CCLX_LOG(::cclx::log_level::warn, __VA_ARGS__)
#define LOG_INFO(...) CCLX_LOG(::cclx::log_level::info, __VA_ARGS__)
#define LOG_DEBUG(...) CCLX_LOG(::cclx::log_level::debug, __VA_ARGS__)
#define LOG_TRACE(...) CCLX_LOG(::cclx::log_level::trace, __VA_ARGS__)

#define CCL_THROW(...) \
    ::cclx::throw_error(__FILE__, __LINE__, __func__, ::cclx::strcat_all(__VA_ARGS__))

#define CCL_THROW_IF_NOT(cond, ...) \
    do { \
        if (!(cond)) \
            ::cclx::throw_error(__FILE__, __LINE__, __func__, \
                                ::cclx::strcat_all("condition ", #cond, " failed. ", ##__VA_ARGS__)); \
    } while (0)

#define CCL_ASSERT(cond, ...) CCL_THROW_IF_NOT(cond, ##__VA_ARGS__)

#define CCL_FATAL(...) \
    do { \
        LOG_ERROR(__VA_ARGS__); \
        std::abort(); \
    } while (0)
