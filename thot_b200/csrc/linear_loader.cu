// The fully connected layer's tensor-core kernels are built into a library of their own,
// libnott_b200_linear.so, next to this one (they are the only part of the tree that instantiates CUTLASS
// collectives, and a host that has no use for them need not ship them).  It is opened on the first call of
// nb2_linear_bias_act_fwd; without it that entry point returns NB2_ERR_UNAVAILABLE and everything else works.
#include <dlfcn.h>
#include <string.h>

#include <mutex>
#include <string>

#include "launchers.h"

namespace nb2 {

namespace {
using PlainFn = int (*)(const void*, const void*, const void*, void*, int64_t, int64_t, int64_t, int, void*, size_t, void*, char*, size_t);
using AuxFn = int (*)(const void*, const void*, const void*, void*, void*, int64_t, int64_t, int64_t, int, void*, size_t, void*, char*, size_t);
struct LinearLib { PlainFn plain = nullptr; AuxFn aux = nullptr; std::string why; };

int anchor;       // any symbol of this library: dladdr() on it gives the library's own path

const LinearLib& linear_lib() {
    static LinearLib lib;
    static std::once_flag once;
    std::call_once(once, [] {
        std::string path = "libnott_b200_linear.so";
        const char* env = getenv("NB2_LINEAR_LIB");
        Dl_info info;
        if (env != nullptr && *env) {
            path = env;
        } else if (dladdr(&anchor, &info) != 0 && info.dli_fname != nullptr) {
            std::string self(info.dli_fname);
            const size_t slash = self.rfind('/');
            if (slash != std::string::npos) path = self.substr(0, slash + 1) + path;
        }
        void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (h == nullptr) {
            const char* e = dlerror();
            lib.why = std::string("the tensor-core linear library could not be loaded (") + (e ? e : path.c_str()) + ")";
            return;
        }
        lib.plain = reinterpret_cast<PlainFn>(dlsym(h, "nb2lin_plain"));
        lib.aux = reinterpret_cast<AuxFn>(dlsym(h, "nb2lin_aux"));
        if (lib.plain == nullptr || lib.aux == nullptr) lib.why = "libnott_b200_linear.so lacks nb2lin_plain / nb2lin_aux";
    });
    return lib;
}
}  // namespace

bool linear_library_present() {
    const LinearLib& l = linear_lib();
    return l.plain != nullptr && l.aux != nullptr;
}

int launch_linear(const void* x, const void* w, const void* bias, void* z_out, void* y, int64_t M, int64_t N, int64_t K, int act,
                  void* workspace, size_t workspace_bytes, cudaStream_t st) {
    const LinearLib& l = linear_lib();
    if (l.plain == nullptr || l.aux == nullptr) {
        set_error("linear: %s", l.why.c_str());
        return NB2_ERR_UNAVAILABLE;
    }
    char msg[400] = "";
    const int rc = z_out != nullptr ? l.aux(x, w, bias, z_out, y, M, N, K, act, workspace, workspace_bytes, (void*)st, msg, sizeof(msg))
                                    : l.plain(x, w, bias, y, M, N, K, act, workspace, workspace_bytes, (void*)st, msg, sizeof(msg));
    if (rc != 0) set_error("%s", msg[0] ? msg : "linear: the tensor-core kernel failed");
    return rc;
}

}  // namespace nb2
