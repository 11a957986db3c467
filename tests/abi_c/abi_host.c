/* The C ABI of libincin_host.so used from a plain C program: no Python, no Rust, no C++ in the caller.
 *
 *   1. incin_cpu_mlp_train: the native tape autograd runs the 784 -> 256 (ReLU) -> 10 MLP for 100 SGD steps and the
 *      loss must fall;
 *   2. a three-rank rendezvous in threads (incin_rdv_connect on 127.0.0.1), an all-gather of one blob per rank over
 *      the control channel, then an orderly shutdown;
 *   3. the reference transport: all-reduce(sum) and all-gather over three ranks' host buffers;
 *   4. the FNV-1a digest of a known string.
 * Prints "ABI_OK" and exits 0 when everything holds; any failure prints what failed and exits 1.
 * Built and run by tests/test_abi_c_cpu.py:  gcc abi_host.c -I csrc/include -L incin_b200/lib -lincin_host -lpthread */
#include <math.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "incin_host.h"

#define CHECK(cond, what)                                   \
  do {                                                      \
    if (!(cond)) {                                          \
      fprintf(stderr, "ABI_FAIL %s (line %d)\n", what, __LINE__); \
      exit(1);                                              \
    }                                                       \
  } while (0)

#define WORLD 3

typedef struct {
  int rank;
  const char* addr;
  int rc_connect, rc_gather, rc_shutdown;
  unsigned char gathered[WORLD * 8];
  long long peer_dev;
} rank_t;

static void* rank_main(void* arg) {
  rank_t* r = (rank_t*)arg;
  int64_t h = 0;
  r->rc_connect = incin_rdv_connect(r->rank, WORLD, r->addr, "abi-c-run", /*local_device=*/10 + r->rank, 8000, &h);
  if (r->rc_connect != 0) return NULL;
  unsigned char mine[8];
  memset(mine, 0x40 + r->rank, sizeof mine);
  r->rc_gather = incin_rdv_allgather(h, mine, 8, r->gathered, 8000);
  r->peer_dev = (long long)incin_rdv_peer_device(h, (r->rank + 1) % WORLD);
  r->rc_shutdown = incin_rdv_shutdown(h, 8000);
  incin_rdv_destroy(h);
  return NULL;
}

int main(int argc, char** argv) {
  const char* addr = argc > 1 ? argv[1] : "127.0.0.1:29777";

  /* 1. native MLP training loop */
  enum { STEPS = 100, NIN = 784, NH = 256, NOUT = 10 };
  float* losses = (float*)malloc(sizeof(float) * STEPS);
  float* params = (float*)malloc(sizeof(float) * (NH * NIN + NH + NOUT * NH + NOUT));
  CHECK(losses && params, "malloc");
  CHECK(incin_cpu_mlp_train(STEPS, 64, NIN, NH, NOUT, 0.01f, 0, losses, params) == 0, "incin_cpu_mlp_train");
  CHECK(isfinite(losses[0]) && isfinite(losses[STEPS - 1]) && losses[STEPS - 1] < losses[0], "MLP loss falls");

  /* 2. rendezvous of three ranks in threads */
  pthread_t th[WORLD];
  rank_t ranks[WORLD];
  for (int i = 0; i < WORLD; ++i) {
    memset(&ranks[i], 0, sizeof ranks[i]);
    ranks[i].rank = i;
    ranks[i].addr = addr;
    CHECK(pthread_create(&th[i], NULL, rank_main, &ranks[i]) == 0, "pthread_create");
  }
  for (int i = 0; i < WORLD; ++i) pthread_join(th[i], NULL);
  for (int i = 0; i < WORLD; ++i) {
    CHECK(ranks[i].rc_connect == 0, "incin_rdv_connect");
    CHECK(ranks[i].rc_gather == 0, "incin_rdv_allgather");
    CHECK(ranks[i].rc_shutdown == 0, "incin_rdv_shutdown");
    for (int r = 0; r < WORLD; ++r)
      for (int b = 0; b < 8; ++b) CHECK(ranks[i].gathered[r * 8 + b] == 0x40 + r, "all-gather content");
    CHECK(ranks[i].peer_dev == 10 + (i + 1) % WORLD, "incin_rdv_peer_device");
  }

  /* 3. reference transport on host memory: dtype 5 = f32 in the library's dtype ids, op 0 = sum */
  float in0[4] = {1, 2, 3, 4}, in1[4] = {10, 20, 30, 40}, in2[4] = {100, 200, 300, 400};
  float out0[12], out1[12], out2[12];
  const void* ins[WORLD] = {in0, in1, in2};
  void* outs[WORLD] = {out0, out1, out2};
  int f32 = -1;
  for (int dt = 0; dt < 8 && f32 < 0; ++dt) {       /* find the id that behaves as f32 (ids are an enum of the library) */
    memset(out0, 0, sizeof out0);
    if (incin_ref_all_reduce(ins, outs, WORLD, 4, dt, 0) == 0 && fabsf(out0[0] - 111.0f) < 1e-5f && fabsf(out0[3] - 444.0f) < 1e-5f) f32 = dt;
  }
  CHECK(f32 >= 0, "incin_ref_all_reduce(sum) over f32");
  CHECK(fabsf(out2[1] - 222.0f) < 1e-5f, "all ranks receive the sum");
  CHECK(incin_ref_all_gather(ins, outs, WORLD, 4, f32) == 0, "incin_ref_all_gather");
  CHECK(out1[0] == 1 && out1[4] == 10 && out1[11] == 400, "all-gather is rank-major");

  /* 4. digest */
  CHECK(incin_fnv1a64("a", 1) == 0xaf63dc4c8601ec8cULL, "FNV-1a 64 of \"a\"");

  printf("ABI_OK f32_id=%d loss %.4f -> %.4f\n", f32, losses[0], losses[STEPS - 1]);
  free(losses);
  free(params);
  return 0;
}
