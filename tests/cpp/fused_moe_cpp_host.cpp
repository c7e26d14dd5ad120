// C++ caller of the ck_tile-shaped host surface (fused_moe_traits / fused_moe_args /
// fused_moe(traits, args, stream)) linked against libfmoe_b200.so.  It reads one problem
// from a flat binary file written by the Python test, runs moe_sorting and fused_moe on the
// device and writes the outputs back, so the test can compare them with the oracle.
//
// File layout (little endian): int32 T, H, I, E, K, quant; then x bf16 [T,H]; w1 [E,2I,H];
// w2 [E,H,I] (2 bytes per element for quant 0, 1 byte otherwise); scales f32 (quant 1:
// [E,2I] and [E,H]); topk_ids i32 [T,K]; topk_weight f32 [T,K].
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "fused_moe.hpp"

#define CK(x)                                                                      \
  do {                                                                             \
    cudaError_t e = (x);                                                           \
    if (e != cudaSuccess) {                                                        \
      std::fprintf(stderr, "CUDA error %s at line %d\n", cudaGetErrorString(e), __LINE__); \
      return 2;                                                                    \
    }                                                                              \
  } while (0)

static std::vector<char> read_exact(FILE* f, size_t n) {
  std::vector<char> v(n);
  if (n && std::fread(v.data(), 1, n, f) != n) { std::fprintf(stderr, "short read\n"); std::exit(3); }
  return v;
}

template <typename T>
static T* to_device(const std::vector<char>& h) {
  void* d = nullptr;
  if (cudaMalloc(&d, h.size() ? h.size() : 1) != cudaSuccess) std::exit(4);
  cudaMemcpy(d, h.data(), h.size(), cudaMemcpyHostToDevice);
  return static_cast<T*>(d);
}

int main(int argc, char** argv) {
  if (argc != 3) { std::fprintf(stderr, "usage: %s problem.bin result.bin\n", argv[0]); return 1; }
  FILE* f = std::fopen(argv[1], "rb");
  if (!f) return 1;
  int32_t dims[6];
  if (std::fread(dims, 4, 6, f) != 6) return 3;
  const int T = dims[0], H = dims[1], I = dims[2], E = dims[3], K = dims[4], quant = dims[5];
  const size_t wb = quant == 0 ? 2 : 1;
  auto hx = read_exact(f, size_t(T) * H * 2);
  auto hw1 = read_exact(f, size_t(E) * 2 * I * H * wb);
  auto hw2 = read_exact(f, size_t(E) * H * I * wb);
  auto hs1 = read_exact(f, quant == 1 ? size_t(E) * 2 * I * 4 : 0);
  auto hs2 = read_exact(f, quant == 1 ? size_t(E) * H * 4 : 0);
  auto hid = read_exact(f, size_t(T) * K * 4);
  auto hwt = read_exact(f, size_t(T) * K * 4);
  std::fclose(f);

  cudaStream_t stream;
  CK(cudaStreamCreate(&stream));

  fused_moe_traits traits;
  traits.prec_w = quant == 0 ? "bf16" : "fp8";
  traits.quant = quant == 0 ? "none" : "token_channel";

  fused_moe_args args;
  args.a_ptr = to_device<void>(hx);
  args.g_ptr = to_device<void>(hw1);
  args.d_ptr = to_device<void>(hw2);
  args.g_scale_ptr = quant ? to_device<float>(hs1) : nullptr;
  args.d_scale_ptr = quant ? to_device<float>(hs2) : nullptr;
  args.topk_ids_ptr = to_device<int32_t>(hid);
  args.topk_weight_ptr = to_device<float>(hwt);
  args.num_tokens = T; args.hidden_size = H; args.intermediate_size = I; args.num_experts = E; args.topk = K;
  void* out = nullptr;
  CK(cudaMalloc(&out, size_t(T) * H * 2));
  args.o_ptr = out;
  const int64_t ws = fused_moe_get_workspace_size(traits, args);
  if (ws < 0) { std::fprintf(stderr, "workspace query failed: %s\n", fmoe_last_error()); return 5; }
  CK(cudaMalloc(&args.ws_ptr, size_t(ws)));
  args.ws_bytes = uint64_t(ws);

  // moe_sorting on its own, as a ck_tile user would call it
  const int64_t cap = fmoe_sort_capacity(T, K, E, 128);
  moe_sorting_args sa;
  int32_t *s_ids, *s_eids, *s_npp;
  float* s_w;
  CK(cudaMalloc(&s_ids, cap * 4)); CK(cudaMalloc(&s_w, cap * 4));
  CK(cudaMalloc(&s_eids, cap / 128 * 4)); CK(cudaMalloc(&s_npp, 4));
  sa.p_topk_ids = args.topk_ids_ptr; sa.p_weights = args.topk_weight_ptr;
  sa.p_sorted_token_ids = s_ids; sa.p_sorted_weights = s_w; sa.p_sorted_expert_ids = s_eids;
  sa.p_total_tokens_post_pad = s_npp;
  sa.tokens = T; sa.unit_size = 128; sa.num_experts = E; sa.topk = K;
  if (moe_sorting(sa, stream_config{stream, false}) < 0) { std::fprintf(stderr, "moe_sorting: %s\n", fmoe_last_error()); return 6; }

  const float ms = fused_moe(traits, args, stream_config{stream, true});   // timed: synchronises
  if (ms < 0) { std::fprintf(stderr, "fused_moe failed (%g): %s\n", ms, fmoe_last_error()); return 7; }
  // an invalid request must come back as an error code, not a crash
  fused_moe_args bad = args;
  bad.o_ptr = nullptr;
  if (fused_moe(traits, bad, stream_config{stream, false}) >= 0) return 8;

  std::vector<char> hout(size_t(T) * H * 2), hsid(cap * 4);
  int32_t npp = 0;
  CK(cudaMemcpy(hout.data(), out, hout.size(), cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(hsid.data(), s_ids, hsid.size(), cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(&npp, s_npp, 4, cudaMemcpyDeviceToHost));
  FILE* g = std::fopen(argv[2], "wb");
  if (!g) return 1;
  std::fwrite(&npp, 4, 1, g);
  std::fwrite(hsid.data(), 1, hsid.size(), g);
  std::fwrite(hout.data(), 1, hout.size(), g);
  std::fclose(g);
  std::printf("fused_moe ok: %.3f ms, num_tokens_post_pad=%d\n", ms, npp);
  return 0;
}
