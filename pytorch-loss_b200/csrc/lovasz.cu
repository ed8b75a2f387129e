// placeholder until the Lovasz pipeline lands
#include "common.cuh"
using namespace b200;
extern "C" size_t b200_lovasz_workspace_bytes(int64_t, int64_t, int64_t, int) { return 0; }
extern "C" int b200_lovasz_forward(const void *, const int64_t *, float *, float *, void *, size_t,
                                   int64_t, int64_t, int64_t, int, int64_t, int, void *) {
    set_error("lovasz: not built yet");
    return B200_ERR_UNSUPPORTED;
}
extern "C" int b200_lovasz_backward(const float *, const void *, const int64_t *, const float *,
                                    void *, int64_t, int64_t, int64_t, int, int64_t, int, void *) {
    set_error("lovasz: not built yet");
    return B200_ERR_UNSUPPORTED;
}
