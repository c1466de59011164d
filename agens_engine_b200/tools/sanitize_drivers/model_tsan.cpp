// The collectives' inbox protocol model (csrc/comm/protocol_model.cpp) under ThreadSanitizer; built and run by
// tools/sanitize.py (tsan-model).
#include <cstdio>
#include <initializer_list>
extern "C" int b2h_comm_model_run(int, int, int, unsigned, int, int, int, int, char*, int);
int main() {
  char rep[256]; int bad = 0;
  for (int ranks : {2, 4, 8}) for (unsigned seed = 0; seed < 3; ++seed) {
    bad += b2h_comm_model_run(ranks, 60, 16, seed, 0, -1, -1, 60000, rep, 256); printf("%s\n", rep);
    bad += b2h_comm_model_run(ranks, 40, 12, seed, 1, -1, -1, 60000, rep, 256); printf("%s\n", rep);
  }
  bad += b2h_comm_model_run(4, 30, 8, 7, 0, 1, 11, 1500, rep, 256); printf("%s\n", rep);
  printf("bad %d\n", bad);
  return bad ? 1 : 0;
}
