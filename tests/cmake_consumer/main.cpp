// Links against the installed library through find_package and calls host-only entry points.
#include <cstdio>

#include "fused_moe.hpp"

int main() {
  fused_moe_traits t;
  fused_moe_args a;
  a.num_tokens = 128; a.hidden_size = 512; a.intermediate_size = 1024; a.num_experts = 8; a.topk = 2;
  const long long bytes = fused_moe_get_workspace_size(t, a);
  std::printf("version %d capacity %lld workspace %lld\n", fmoe_version(),
              static_cast<long long>(fmoe_sort_capacity(128, 2, 8, 128)), bytes);
  return (fmoe_version() >= 100 && bytes > 0) ? 0 : 1;
}
