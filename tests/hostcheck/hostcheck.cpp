// Host-side half of the backend (wire-format parser, data-parallel rewrite, lowering, CUDA source generation)
// as a stand-alone program, so that it can be built with AddressSanitizer + UndefinedBehaviorSanitizer and fed
// serialised programs from files.  No CUDA involved: the sources compiled in are plain C++.
//
//   hostcheck <flags> <world> <shard_batch> <blob files ...>
//
// flags: bit 0 no fusion, bit 1 fold small sums, bit 2 correctly rounded division.
// Malformed blobs must be rejected with an exception (counted), never crash.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iterator>
#include <vector>

#include "adb_ir.hpp"
#include "adb_lower.hpp"
#include "adb_shard.hpp"

int main(int argc, char** argv) {
    if (argc < 5) return 2;
    const unsigned flags = unsigned(std::atoi(argv[1]));
    const int world = std::atoi(argv[2]);
    const long long batch = std::atoll(argv[3]);
    size_t kernels = 0, rejected = 0, fused = 0;
    for (int f = 4; f < argc; f++) {
        std::ifstream in(argv[f], std::ios::binary);
        std::vector<uint8_t> blob((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
        for (int rank = 0; rank < world; rank++) {
            try {
                adb::Program prog = adb::parse_program(blob.data(), blob.size());
                adb::LowerOptions opt;
                opt.no_fusion = flags & 1;
                opt.fuse_small_sums = flags & 2;
                opt.exact_div = flags & 4;
                opt.rank = rank;
                opt.world = world;
                if (world > 1 && batch) adb::shard_program(prog, rank, world, batch);
                adb::Plan plan;
                adb::lower_program(prog, plan, opt);
                adb::generate_kernels(plan);
                for (auto& k : plan.kernels) {
                    kernels += !k.dead;
                    fused += k.reds.size();
                }
                std::string listing = adb::dump_plan(plan, true);
                if (listing.empty()) return 3;
            } catch (const std::exception& e) {
                rejected++;
            }
        }
    }
    std::printf("files=%d kernels=%zu fused_sums=%zu rejected=%zu\n", argc - 4, kernels, fused, rejected);
    return 0;
}
