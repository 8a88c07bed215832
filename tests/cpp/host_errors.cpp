// Builds against maxuna_b200/host/laguna_moe.hpp and liblmoe.so; exercises argument errors
// that are reported before any CUDA call (so it runs without a GPU). Prints "ok" on success.
#include <cstdio>
#include <cstring>

#include "../../maxuna_b200/host/laguna_moe.hpp"

int main() {
    using namespace laguna;
    ExpertStack st;
    // size mismatch: an Err, not a crash
    Result r = ExpertStack::view(GgmlDType::Q4K, 4, 8, 256, (const void *)4096, 7 * 144, 0, st);
    if (r.ok() || r.message.find("does not match") == std::string::npos) { std::printf("bad: %s\n", r.message.c_str()); return 1; }
    r = ExpertStack::view(GgmlDType::Q4K, 4, 8, 256, (const void *)4096, 4 * 8 * 144, 0, st);
    if (!r.ok()) { std::printf("bad view: %s\n", r.message.c_str()); return 1; }
    // k mismatch (src/ops/mv_id.rs:137-145 of the reference: an error, not a fault)
    r = ops::mul_mv_id(st, (const float *)4096, 1, 1, 128, (const uint32_t *)4096, 1, 2, (float *)4096, nullptr);
    if (r.ok() || r.message.find("does not match expert stack k") == std::string::npos) { std::printf("bad: %s\n", r.message.c_str()); return 1; }
    // combine guard
    r = ops::combine((const float *)4096, nullptr, (const float *)4096, 1, 200, 8, (float *)4096, nullptr);
    if (r.ok()) return 1;
    if (!ops::supported(GgmlDType::Q6K, 10)) return 1;
    // the layer entry without a layer handle: an Err
    MoeBlock blk;
    r = blk.layer_forward((const float *)4096, (const float *)4096, 1e-6f, 1, (float *)8192, nullptr, 0, nullptr);
    if (r.ok() || r.message.find("layer is NULL") == std::string::npos) { std::printf("bad: %s\n", r.message.c_str()); return 1; }
    if (blk.layer_workspace_bytes(16) != 0) return 1;
    std::printf("ok\n");
    return 0;
}
