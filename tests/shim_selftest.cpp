// Self-test of the stand-in SYCL runtime (oracle/ref_shim/sycl/sycl.hpp) that the reference's sources
// are compiled against for the oracle pin: the properties the pin relies on, checked directly.
//   1. barriers: every work-item of a group reaches a barrier before any leaves it (a shared-memory
//      tree reduction written with explicit barriers gives the tree's result);
//   2. reduce_over_group over a work-group and over a sub-group of 16 adds in the balanced tree
//      t[i] += t[i + w], w = n/2 .. 1 (values chosen so that every other order rounds differently);
//   3. nd_range<2>: get_local_id(1) runs fastest, groups are enumerated the same way;
//   4. a work-item that returns early does not block the barriers of the others.
#include <cmath>
#include <cstdio>
#include <vector>

#include <sycl/sycl.hpp>

static float tree(std::vector<float> t) {
    for (size_t w = t.size() / 2; w >= 1; w /= 2)
        for (size_t i = 0; i < w; ++i) t[i] = t[i] + t[i + w];
    return t[0];
}

int main() {
    sycl::queue q;
    // values spanning many binades: float addition order matters
    std::vector<float> v(256);
    for (int i = 0; i < 256; ++i) v[i] = std::ldexp(1.0f + 0.37f * (float)((i * 37) % 11), (i * 7) % 23 - 11) * ((i % 3) ? 1.0f : -1.0f);
    float seq = 0.0f;
    for (float x : v) seq += x;
    const float want = tree(v);
    if (want == seq) { std::printf("test vector does not separate the orders\n"); return 10; }

    float got_manual = 0.0f, got_reduce = 0.0f;
    std::vector<float> got_sg(16, 0.0f);
    const float* vp = v.data();
    float* gm = &got_manual;
    float* gr = &got_reduce;
    float* gs = got_sg.data();
    q.submit([&](sycl::handler& cgh) {
        sycl::local_accessor<float, 1> sh(sycl::range<1>(256), cgh);
        cgh.parallel_for(sycl::nd_range<1>(256, 256), [=](sycl::nd_item<1> item) {
            const int lid = (int)item.get_local_id(0);
            sh[lid] = vp[lid];
            item.barrier(sycl::access::fence_space::local_space);
            for (int stride = 128; stride > 0; stride >>= 1) {
                if (lid < stride) sh[lid] += sh[lid + stride];
                item.barrier(sycl::access::fence_space::local_space);
            }
            if (lid == 0) *gm = sh[0];
            const float r = sycl::reduce_over_group(item.get_group(), vp[lid], sycl::plus<float>());
            if (lid == 5) *gr = r;
            const float s = sycl::reduce_over_group(item.get_sub_group(), vp[lid], sycl::plus<>());
            if (lid % 16 == 3) gs[lid / 16] = s;
        });
    });
    if (got_manual != want) { std::printf("barrier reduction %a != %a\n", got_manual, want); return 1; }
    if (got_reduce != want) { std::printf("reduce_over_group %a != %a\n", got_reduce, want); return 2; }
    for (int g = 0; g < 16; ++g) {
        std::vector<float> part(v.begin() + 16 * g, v.begin() + 16 * g + 16);
        if (got_sg[g] != tree(part)) { std::printf("sub-group %d\n", g); return 3; }
    }
    // nd_range<2>: local id 1 fastest; each item records its linearised position
    std::vector<int> seen(6 * 8, -1);
    int* sp = seen.data();
    q.submit([&](sycl::handler& cgh) {
        cgh.parallel_for(sycl::nd_range<2>(sycl::range<2>(6, 8), sycl::range<2>(3, 4)), [=](sycl::nd_item<2> item) {
            const int g0 = (int)item.get_group(0), g1 = (int)item.get_group(1);
            const int l0 = (int)item.get_local_id(0), l1 = (int)item.get_local_id(1);
            const int row = g0 * 3 + l0, col = g1 * 4 + l1;
            sp[row * 8 + col] = (int)item.get_local_linear_id() == l0 * 4 + l1 ? (int)(item.get_global_id(0) * 8 + item.get_global_id(1)) : -2;
        });
    });
    for (int i = 0; i < 48; ++i)
        if (seen[i] != i) { std::printf("nd_range<2> mapping at %d: %d\n", i, seen[i]); return 4; }
    // early return of some items must not block the others' barriers
    int after = 0;
    int* ap = &after;
    q.submit([&](sycl::handler& cgh) {
        cgh.parallel_for(sycl::nd_range<1>(64, 32), [=](sycl::nd_item<1> item) {
            if (item.get_group(0) == 1) return;  // a whole group leaves (as decode_prepare_qkv's kv test does)
            item.barrier(sycl::access::fence_space::local_space);
            if (item.get_local_id(0) == 0) *ap += 1;
        });
    });
    if (after != 1) { std::printf("early return\n"); return 5; }
    // plain 2-D range: last dimension fastest
    std::vector<int> order;
    std::vector<int>* op = &order;
    q.parallel_for(sycl::range<2>(2, 3), [=](sycl::id<2> idx) { op->push_back((int)(idx[0] * 3 + idx[1])); });
    for (int i = 0; i < 6; ++i)
        if (order[i] != i) { std::printf("range<2> order\n"); return 6; }
    std::printf("shim ok\n");
    return 0;
}
