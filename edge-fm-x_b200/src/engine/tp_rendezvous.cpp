#include "tp_rendezvous.h"

#include <sys/stat.h>

#include <chrono>
#include <cstdio>
#include <fstream>
#include <thread>

#include "edge-fm/core.h"

namespace edge_fm {

TpRendezvous::TpRendezvous(const std::string& dir, int rank, int world, double timeout_s)
    : dir_(dir), rank_(rank), world_(world), timeout_s_(timeout_s) {
    if (dir_.empty()) throw ConfigurationError("tensor parallel engines need runtime.tp_rendezvous (or EFM_TP_RENDEZVOUS): a fresh directory shared by the ranks");
    if (rank_ < 0 || rank_ >= world_) throw ConfigurationError("tensor parallel rank out of range");
    struct stat st;
    if (stat(dir_.c_str(), &st) != 0) {
        if (mkdir(dir_.c_str(), 0700) != 0 && stat(dir_.c_str(), &st) != 0)      // another rank may have created it meanwhile
            throw ConfigurationError("cannot create the rendezvous directory " + dir_);
    } else if (!S_ISDIR(st.st_mode)) {
        throw ConfigurationError("rendezvous path is not a directory: " + dir_);
    }
}

void TpRendezvous::publish(const std::string& file, const std::vector<char>& bytes) const {
    const std::string path = dir_ + "/" + file, tmp = path + ".tmp" + std::to_string(rank_);
    {
        std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
        if (!f.is_open()) throw ConfigurationError("cannot write " + tmp);
        f.write(bytes.data(), (std::streamsize)bytes.size());
    }
    if (std::rename(tmp.c_str(), path.c_str()) != 0) throw ConfigurationError("cannot publish " + path);
}

std::vector<char> TpRendezvous::await(const std::string& file) const {
    const std::string path = dir_ + "/" + file;
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        std::ifstream f(path, std::ios::binary);
        if (f.is_open()) return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
        const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (waited > timeout_s_)
            throw ConfigurationError("tensor parallel rendezvous timed out waiting for " + path + " (is every rank running, and is the directory fresh?)");
        std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
}

std::vector<char> TpRendezvous::broadcast_from_root(const std::string& name, const std::vector<char>& bytes) {
    if (rank_ == 0) {
        publish(name, bytes);
        return bytes;
    }
    return await(name);
}

std::vector<std::vector<char>> TpRendezvous::all_gather(const std::string& name, const std::vector<char>& bytes) {
    publish(name + "." + std::to_string(rank_), bytes);
    std::vector<std::vector<char>> out((size_t)world_);
    for (int r = 0; r < world_; ++r) out[(size_t)r] = r == rank_ ? bytes : await(name + "." + std::to_string(r));
    return out;
}

void TpRendezvous::barrier(const std::string& name) { (void)all_gather(name, std::vector<char>(1, 1)); }

}  // namespace edge_fm
