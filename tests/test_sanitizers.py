"""Host-side sanitizer runs (compute-sanitizer is not available for the device code, so the
host parts that can be checked this way are): the C-ABI's validation / planning code and the
CPU oracle, each built with -fsanitize=address,undefined and run on edge-case inputs."""
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SAN = ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer", "-g", "-O1"]


def _env():
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX", "LD_PRELOAD")}
    env["ASAN_OPTIONS"] = "detect_leaks=1:abort_on_error=0"
    return env


def test_validation_and_planning_under_asan_ubsan(tmp_path):
    exe = tmp_path / "plan_sanitize"
    subprocess.run(["g++", "-std=c++17", *SAN, "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "plan_sanitize.cpp"), "-o", str(exe)], check=True, env=_env())
    r = subprocess.run([str(exe)], capture_output=True, text=True, env=_env())
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.strip().endswith("ok")


ORACLE_DRIVER = r"""
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
int orc_route(const float*, int, int, int, int, int32_t*, float*);
int64_t orc_sort_capacity(int64_t, int64_t, int64_t, int64_t);
int orc_moe_sorting(const int32_t*, const float*, int, int, int, int, int32_t*, float*, int32_t*, int32_t*, int32_t*, int32_t*);
void orc_f32_to_bf16(const float*, uint16_t*, int64_t);
void orc_quant_rows_e4m3_ex(const float*, int64_t, int64_t, int64_t, int, uint8_t*, float*);
void orc_quant_blocks_e4m3_ex(const float*, int64_t, int64_t, int, uint8_t*, float*);
int orc_fused_moe_ex2(int, int, int, int, int, int, int, int, const uint16_t*, const void*, const void*, const float*,
                      const float*, const int32_t*, const float*, const int32_t*, int, uint16_t*, int);
static float rnd(uint32_t* s) { *s = *s * 1664525u + 1013904223u; return ((*s >> 8) / 8388608.0f) - 1.0f; }
int main(void) {
  const int T = 37, H = 256, I = 128, E = 5, K = 3;
  uint32_t seed = 7;
  float* logits = malloc(sizeof(float) * T * E);
  for (int i = 0; i < T * E; ++i) logits[i] = rnd(&seed);
  int32_t* ids = malloc(sizeof(int32_t) * T * K);
  float* w = malloc(sizeof(float) * T * K);
  if (orc_route(logits, T, E, K, 1, ids, w)) return 2;
  ids[4] = -1; ids[7] = E + 9;                       /* invalid ids are dropped */
  int64_t cap = orc_sort_capacity(T, K, E, 128);
  int32_t* st = malloc(4 * cap); float* sw = malloc(4 * cap); int32_t* sr = malloc(4 * cap);
  int32_t* se = malloc(4 * (cap / 128)); int32_t npp; int32_t* cum = malloc(4 * (E + 1));
  orc_moe_sorting(ids, w, T, K, E, 128, st, sw, sr, se, &npp, cum);
  orc_moe_sorting(ids, w, 0, K, E, 128, st, NULL, NULL, NULL, NULL, NULL);   /* empty batch, optional outputs */
  float* xf = malloc(sizeof(float) * T * H); uint16_t* x = malloc(2 * T * H);
  for (int i = 0; i < T * H; ++i) xf[i] = rnd(&seed);
  for (int i = 0; i < H; ++i) xf[3 * H + i] = 0.0f;   /* an all-zero row */
  orc_f32_to_bf16(xf, x, (int64_t)T * H);
  float* w1f = malloc(sizeof(float) * E * 2 * I * H); float* w2f = malloc(sizeof(float) * E * H * I);
  for (int i = 0; i < E * 2 * I * H; ++i) w1f[i] = 0.02f * rnd(&seed);
  for (int i = 0; i < E * H * I; ++i) w2f[i] = 0.02f * rnd(&seed);
  uint16_t* out = malloc(2 * T * H);
  for (int quant = 0; quant <= 3; ++quant) {
    void *w1, *w2; float *s1 = NULL, *s2 = NULL;
    if (quant == 0) {
      w1 = malloc(2 * E * 2 * I * H); w2 = malloc(2 * E * H * I);
      orc_f32_to_bf16(w1f, w1, (int64_t)E * 2 * I * H); orc_f32_to_bf16(w2f, w2, (int64_t)E * H * I);
    } else if (quant == 1) {
      w1 = malloc(E * 2 * I * H); w2 = malloc(E * H * I);
      s1 = malloc(4 * E * 2 * I); s2 = malloc(4 * E * H);
      orc_quant_rows_e4m3_ex(w1f, E * 2 * I, H, H, 0, w1, s1); orc_quant_rows_e4m3_ex(w2f, E * H, I, I, 0, w2, s2);
    } else {
      w1 = malloc(E * 2 * I * H); w2 = malloc(E * H * I);
      s1 = malloc(4 * (E * 2 * I / 128) * (H / 128)); s2 = malloc(4 * (E * H / 128) * (I / 128));
      orc_quant_blocks_e4m3_ex(w1f, E * 2 * I, H, quant == 3, w1, s1);
      orc_quant_blocks_e4m3_ex(w2f, E * H, I, quant == 3, w2, s2);
    }
    for (int pb = 0; pb <= 1; ++pb)
      if (orc_fused_moe_ex2(T, H, I, E, K, quant, 0, pb, x, w1, w2, s1, s2, ids, w, NULL, 0, out, 2)) return 3;
    int32_t sel[3] = {0, 3, T - 1};
    if (orc_fused_moe_ex2(T, H, I, E, K, quant, 0, 0, x, w1, w2, s1, s2, ids, w, sel, 3, out, 1)) return 4;
    free(w1); free(w2); free(s1); free(s2);
  }
  free(logits); free(ids); free(w); free(st); free(sw); free(sr); free(se); free(cum);
  free(xf); free(x); free(w1f); free(w2f); free(out);
  printf("ok\n");
  return 0;
}
"""


def test_cpu_oracle_under_asan_ubsan(tmp_path):
    drv = tmp_path / "driver.c"
    drv.write_text(ORACLE_DRIVER)
    exe = tmp_path / "oracle_sanitize"
    subprocess.run(["gcc", "-std=gnu11", *SAN, "-fopenmp", os.path.join(ROOT, "oracle", "fmoe_oracle.c"), str(drv),
                    "-lm", "-o", str(exe)], check=True, env=_env())
    r = subprocess.run([str(exe)], capture_output=True, text=True, env=_env())
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.strip().endswith("ok")
