// Host-only check of the C++ shim: split_CSR<int> and build_part<int> called exactly as the
// reference's drivers call them (src/mgg_np_div_mem.cu:94, src/test_neighbor_part.cu), printing every
// returned array.  tests/test_compat_host.py compiles this file against the built library, runs it
// without a GPU and compares the printed arrays with the Python API and the known answers.
#include <cstdio>
#include <vector>

#include "mgg_compat.hpp"

static void show(const char* tag, const std::vector<int>& v) {
    printf("%s", tag);
    for (int x : v) printf(" %d", x);
    printf("\n");
}

int main() {
    // split: the small case
    std::vector<int> ptr = {0, 2, 3, 5, 6}, col = {1, 2, 0, 0, 3, 2};
    auto s = split_CSR<int>(ptr, col, 0, 2);
    show("split_small_local_ptr", s[0]);
    show("split_small_remote_ptr", s[1]);
    show("split_small_local_col", s[2]);
    show("split_small_remote_col", s[3]);

    // split: a 60-node graph from a linear congruential sequence, middle shard of three
    std::vector<int> p2 = {0}, c2;
    unsigned state = 12345u;
    for (int i = 0; i < 60; i++) {
        state = state * 1664525u + 1013904223u;
        const int deg = (int)((state >> 24) % 9);
        for (int k = 0; k < deg; k++) {
            state = state * 1664525u + 1013904223u;
            c2.push_back((int)((state >> 16) % 60));
        }
        p2.push_back((int)c2.size());
    }
    show("lcg_ptr", p2);
    show("lcg_col", c2);
    auto t = split_CSR<int>(p2, c2, 20, 40);
    show("split_lcg_local_ptr", t[0]);
    show("split_lcg_remote_ptr", t[1]);
    show("split_lcg_local_col", t[2]);
    show("split_lcg_remote_col", t[3]);

    // build_part: the small case and the corner case whose last node has no edges
    std::vector<int> ip = {0, 3, 5, 6};
    auto b = build_part<int>("part", ip, 3, 2);
    show("part_small_partPtr", b[0]);
    show("part_small_part2Node", b[1]);
    show("part_small_node2Part", b[2]);
    std::vector<int> ip2 = {0, 3, 5, 5};
    auto b2 = build_part<int>("corner", ip2, 3, 2);
    show("part_corner_partPtr", b2[0]);
    show("part_corner_part2Node", b2[1]);
    show("part_corner_node2Part", b2[2]);
    auto b3 = build_part<int>("lcg", p2, 60, 4);
    show("part_lcg_partPtr", b3[0]);
    show("part_lcg_part2Node", b3[1]);
    show("part_lcg_node2Part", b3[2]);
    return 0;
}
