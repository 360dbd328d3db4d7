// Drives the reference project's own page allocator (paging::PageAllocator, src/core/paging/paged_kv_cache.h:47-71)
// through a seeded random sequence of sequence operations and writes the operations, the free count and the touched sequence's block table after each
// to a JSON file: the anchor of tests/test_allocator_vs_reference.py.  The reference's SequenceManager needs a device
// in its constructor, so its three page rules are applied here by hand around the reference's allocator: a new page
// exactly when the length reaches a page boundary (paged_kv_cache.h:145-153), destroy = decref of every page in table
// order (136-140), truncate = decref from the back (196-208).  Built and run by make_allocator_golden.sh.
#include "core/paging/paged_kv_cache.h"
#include <cstdio>
#include <map>
#include <random>
#include <string>
#include <vector>

using blackwell::paging::PageAllocator;
using blackwell::paging::PageId;

int main(int argc, char** argv) {
    if (argc < 2) { std::fprintf(stderr, "usage: make_allocator_golden <out.json>\n"); return 2; }
    const int page = blackwell::paging::PAGE_SIZE, total = 24;
    PageAllocator alloc(total);
    std::map<int, std::pair<std::vector<PageId>, int>> seqs;   // id -> (pages, length)
    std::mt19937 rng(20240607);
    std::FILE* f = std::fopen(argv[1], "w");
    std::fprintf(f, "{\"page_size\": %d, \"num_pages\": %d, \"ops\": [\n", page, total);
    int next_id = 0;
    bool first = true;
    for (int step = 0; step < 300; ++step) {
        const int kind = (int)(rng() % 10);
        std::string op; int id = -1, arg = 0;
        if (seqs.empty() || (kind < 2 && seqs.size() < 6)) {
            id = next_id++; seqs[id] = {{}, 0}; op = "create";
        } else {
            auto it = seqs.begin(); std::advance(it, rng() % seqs.size());
            id = it->first;
            auto& pages = it->second.first; int& len = it->second.second;
            if (kind < 7) {                                   // append up to 40 tokens, as far as pages exist
                op = "append"; arg = 1 + (int)(rng() % 40);
                int done = 0;
                for (; done < arg; ++done) {
                    if ((int)pages.size() == len / page) {
                        if (alloc.free_pages() == 0) break;
                        pages.push_back(alloc.allocate());
                    }
                    ++len;
                }
                arg = done;
                if (arg == 0) continue;
            } else if (kind < 9) {                            // truncate to a shorter length
                op = "truncate"; arg = len ? (int)(rng() % (len + 1)) : 0;
                const int keep_blocks = (arg + page - 1) / page;
                while ((int)pages.size() > keep_blocks) { alloc.decref(pages.back()); pages.pop_back(); }
                if (arg < len) len = arg;
            } else {
                op = "destroy";
                for (PageId p : pages) alloc.decref(p);
                seqs.erase(it);
            }
        }
        // after the operation: the free count and the block table of the sequence it touched
        std::fprintf(f, "%s {\"op\": \"%s\", \"seq\": %d, \"arg\": %d, \"free\": %d, \"table\": [", first ? "" : ",\n",
                     op.c_str(), id, arg, alloc.free_pages());
        first = false;
        if (seqs.count(id)) {
            const auto& pg = seqs[id].first;
            for (size_t i = 0; i < pg.size(); ++i) std::fprintf(f, "%s%d", i ? ", " : "", pg[i]);
        }
        std::fprintf(f, "]}");
    }
    std::fprintf(f, "\n]}\n");
    std::fclose(f);
    return 0;
}
