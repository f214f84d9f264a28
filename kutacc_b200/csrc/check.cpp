// Error flag, last-error text, version record.
#include <cstring>
#include <iostream>
#include <mutex>

#include "common.h"

namespace kutacc {
bool kutacc_check_err_set = false;
static std::string g_last_error;
static std::mutex g_err_mutex;

void check_fail(const char *func, const char *file, int line, const std::string &msg)
{
    std::ostringstream os;
    os << "KUTACC_CHECK fail in " << func << " at " << file << ":" << line << " , " << msg << "\n\n";
    std::cerr << os.str();
    std::lock_guard<std::mutex> lk(g_err_mutex);
    g_last_error = msg;
    kutacc_check_err_set = true;
}
}  // namespace kutacc

extern "C" {

int kutacc_b200_error_set(void) { return kutacc::kutacc_check_err_set ? 1 : 0; }

int kutacc_b200_last_error(char *buf, size_t cap)
{
    std::lock_guard<std::mutex> lk(kutacc::g_err_mutex);
    if (buf && cap) {
        std::strncpy(buf, kutacc::g_last_error.c_str(), cap - 1);
        buf[cap - 1] = 0;
    }
    return kutacc::kutacc_check_err_set ? 1 : 0;
}

void kutacc_b200_clear_error(void)
{
    std::lock_guard<std::mutex> lk(kutacc::g_err_mutex);
    kutacc::kutacc_check_err_set = false;
    kutacc::g_last_error.clear();
}

// Version record (reference: src/version/version.cpp:15-35).
int kutacc_get_version(kutacc_version_t *version)
{
    if (version == nullptr) return KUTACC_ERROR;
    version->product_name = "Kunpeng HPCKit";
    version->product_version = "26.1.RC1";
    version->component_name = "KuTACC";
    version->component_version = "26.1.RC1-b200";
    version->component_abi_version = "1";
    version->component_appendinfo = "nvcc sm_100a";
    return KUTACC_OK;
}

}  // extern "C"
