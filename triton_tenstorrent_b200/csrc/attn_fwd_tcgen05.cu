#include "launch.h"
namespace b200k {
int attn_supported(int D, int N_CTX) { return 0; }
int attn_fwd_bf16(const AttnArgs& a, cudaStream_t s) { return set_error(B200K_ERR_UNSUPPORTED, "attention: not built yet"); }
}
