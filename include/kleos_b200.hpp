// C++ host-side mirror of the reference's entry points on top of the C ABI in kleos_b200.h.
//
// Same names, argument meaning and error behaviour as the inline host functions a caller of
// the reference uses (namespace kleos):
//   initialize()                         csrc/include/kleos/bootstrap.cuh:532-547
//   finalize()                           bootstrap.cuh:561-588
//   getRank()                            bootstrap.cuh:555-559
//   setDevice()                          bootstrap.cuh:549-553
//   moe::forwardHost(iP, oP)             moe/moe.cuh:186-205
//   moe::forwardHostBench<skip, trials>  moe/moe.cuh:146-184
// so that a driver written against the reference (csrc/main.cu:12-73) compiles against this
// header unchanged apart from the include and the buffer sizes, which the reference takes from
// compile-time constants and this library reports at run time (layerInfo()).
//
// Error behaviour: like the reference (debug.cuh:19-43) every failure prints what went wrong
// and ends the process.  Callers that want status codes use the C ABI directly.
//
// Bootstrap: the reference is started by an MPI / PMI launcher and finds its peers through
// nvshmem_init() (bootstrap.cuh:295).  Here rank and world size are read from the launcher's
// environment (RANK / WORLD_SIZE, OMPI_COMM_WORLD_*, PMI_*, SLURM_*), and the 128-byte NCCL
// id that rank 0 creates reaches the other ranks of the node through a file (KLEOS_ID_FILE, or
// a name derived from the launcher's port or job id and its process id in the temporary
// directory).
#pragma once

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <ctime>
#include <fstream>
#include <initializer_list>
#include <string>
#include <thread>

#include <sys/stat.h>
#include <unistd.h>

#include "kleos_b200.h"

namespace kleos {

namespace detail {
[[noreturn]] inline void die(const char* what, int rc) {
    std::fprintf(stderr, "Error: %s: %s\n", what, kleos_error_string(rc));
    std::fflush(stderr);
    std::exit(1);
}
inline void check(int rc, const char* what) {
    if (rc != KLEOS_OK) die(what, rc);
}
inline int env_int(std::initializer_list<const char*> names, int fallback) {
    for (const char* n : names)
        if (const char* v = std::getenv(n)) return std::atoi(v);
    return fallback;
}
inline bool& initialised() {
    static bool flag = false;
    return flag;
}
inline std::string& id_path() {
    static std::string p;
    return p;
}
}  // namespace detail

// How this process was launched; fill it by hand or with launchFromEnv().
struct Launch {
    int rank = 0, world = 1;
    std::string config = "kleos_config.json";  // same file the reference's build reads
    std::string id_file;                        // rendezvous file for the NCCL id (world > 1)
    int id_timeout_s = 120;
};

inline Launch launchFromEnv() {
    Launch l;
    l.rank = detail::env_int({"RANK", "OMPI_COMM_WORLD_RANK", "PMI_RANK", "SLURM_PROCID"}, 0);
    l.world = detail::env_int({"WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", "PMI_SIZE", "SLURM_NTASKS"}, 1);
    if (const char* c = std::getenv("KLEOS_CONFIG")) l.config = c;
    if (const char* f = std::getenv("KLEOS_ID_FILE")) {
        l.id_file = f;
    } else {
        // the launcher's process id is part of the name, so the file a crashed earlier launch
        // left behind (same port, same job) is never mistaken for this launch's
        const char* tmp = std::getenv("TMPDIR");
        const char* tag = std::getenv("MASTER_PORT");
        if (!tag) tag = std::getenv("SLURM_JOB_ID");
        l.id_file = std::string(tmp ? tmp : "/tmp") + "/kleos_id_" + (tag ? std::string(tag) + "_" : std::string()) +
                    std::to_string(static_cast<long>(getppid()));
    }
    return l;
}

namespace detail {
// Seconds since the epoch of the file's last modification, or -1 when it does not exist.
inline long long mtime_of(const std::string& path) {
    struct stat st;
    return ::stat(path.c_str(), &st) == 0 ? static_cast<long long>(st.st_mtime) : -1;
}
}  // namespace detail

// Rank 0 creates the 128-byte NCCL id and publishes it in l.id_file (written under another name,
// then renamed, so that a reader never sees half of it); every other rank polls for the file.
inline void exchangeId(const Launch& l, unsigned char (&id)[128]) {
    if (l.rank == 0) {
        std::remove(l.id_file.c_str());  // whatever an earlier launch left under this name
        detail::check(kleos_get_unique_id(id), "kleos_get_unique_id");
        const std::string tmp = l.id_file + ".part";
        {
            std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
            f.write(reinterpret_cast<const char*>(id), sizeof(id));
        }
        if (std::rename(tmp.c_str(), l.id_file.c_str()) != 0) {
            std::fprintf(stderr, "Error: cannot publish the NCCL id at %s\n", l.id_file.c_str());
            std::exit(1);
        }
        detail::id_path() = l.id_file;
        return;
    }
    // A file last written well before this process started belongs to an earlier launch (one
    // that crashed before finalize() removed it): ranks of one launch start within the waiting
    // time of one another, so anything older than that is ignored until rank 0 replaces it.
    const long long oldest = static_cast<long long>(std::time(nullptr)) - l.id_timeout_s;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(l.id_timeout_s);
    for (;;) {
        std::ifstream f(l.id_file, std::ios::binary);
        if (f && detail::mtime_of(l.id_file) >= oldest && f.read(reinterpret_cast<char*>(id), sizeof(id)) &&
            f.gcount() == (std::streamsize)sizeof(id))
            return;
        if (std::chrono::steady_clock::now() > deadline) {
            std::fprintf(stderr, "Error: rank %d waited %d s for the NCCL id at %s\n", l.rank,
                         l.id_timeout_s, l.id_file.c_str());
            std::exit(1);
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(20));
    }
}

inline void initialize(const Launch& l) {
    if (detail::initialised()) {
        std::fprintf(stderr, "Error: Already Initialized\n");
        std::quick_exit(EXIT_FAILURE);
    }
    unsigned char id[128] = {};
    if (l.world > 1) exchangeId(l, id);
    detail::check(kleos_initialize(l.config.c_str(), l.rank, l.world, l.world > 1 ? id : nullptr),
                  "kleos_initialize");
    detail::initialised() = true;
}

// Should be called before loading the model (bootstrap.cuh:531-532).
inline void initialize() { initialize(launchFromEnv()); }

inline void finalize() {
    if (!detail::initialised()) {
        std::fprintf(stderr, "Error: Not initialized!\n");
        std::quick_exit(EXIT_FAILURE);
    }
    detail::check(kleos_finalize(), "kleos_finalize");
    detail::initialised() = false;
    if (!detail::id_path().empty()) {
        std::remove(detail::id_path().c_str());
        detail::id_path().clear();
    }
}

inline unsigned getRank() {
    const int r = kleos_get_rank();
    if (r < 0) detail::die("getRank", r);
    return static_cast<unsigned>(r);
}

// The reference re-selects the rank's device here (bootstrap.cuh:549-553); this library picks
// the device inside kleos_initialize (rank modulo the visible devices, or the one requested with
// kleos_set_device before it) and every entry point runs on it, so only the state is checked.
inline void setDevice() {
    if (!detail::initialised()) {
        std::fprintf(stderr, "Error: Not initialized!\n");
        std::quick_exit(EXIT_FAILURE);
    }
}

// Run-time counterpart of the reference's compile-time ACC constants (types.cuh:442-513):
// S, H, I (the reference's P), E, PX, local experts, packed buffer sizes in elements.
inline kleos_layer_info layerInfo() {
    kleos_layer_info info{};
    detail::check(kleos_get_info(&info), "kleos_get_info");
    return info;
}

namespace moe {

inline void forwardHost(const void* iP, void* oP) {
    detail::check(kleos_forward(iP, oP, nullptr), "kleos_forward");
}

template <unsigned skip = 50, unsigned trials = 100>
inline void forwardHostBench(const void* iP, void* oP, float& duration) {
    detail::check(kleos_forward_bench(iP, oP, static_cast<int>(skip), static_cast<int>(trials), &duration),
                  "kleos_forward_bench");
}

}  // namespace moe
}  // namespace kleos
