// torch bindings of the flash-attention kernels (filled in by flash_attn.cu).
#include <torch/library.h>
void register_attn_ops(torch::Library& m) { (void)m; }
