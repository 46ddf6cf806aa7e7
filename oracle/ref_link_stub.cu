// Link stub used only when the reference project's src/demo.cu is compiled into
// the checker library oracle/_ref/libref_cpu.so.  That file defines the CPU
// attention the tests trust as ground truth, but it also contains a main() that
// calls transformer::launch_flash_attention (src/demo.cu:301,309), so the shared
// object needs a definition of that symbol to link.  The checker never calls it:
// reaching it means someone routed GPU work through the oracle, which is a bug.
#include <cstdio>
#include <cstdlib>
#include "flash_attention.h"   // the reference's own header, via -I<reference>/include

namespace transformer {
void launch_flash_attention(const FlashAttentionParams&) {
    std::fprintf(stderr, "oracle/_ref/libref_cpu.so: launch_flash_attention is a link stub; "
                         "the CPU oracle must not be used to launch GPU work\n");
    std::abort();
}
}  // namespace transformer
