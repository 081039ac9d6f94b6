// Driver for the host-side native code under the compiler's sanitizers (tests/test_host_sanitizers.py
// builds it once with -fsanitize=thread and once with -fsanitize=address,undefined, together with
// csrc/cpu/protocol_sim.cpp and csrc/cpu/micrograd.cpp). It drives the cross-rank signalling protocol
// with one thread per rank (clean steps across the 2^32 epoch wrap, a peer that stays silent, the
// last-one-out counter) and the micrograd engine (graph build, backward, release, reuse of node slots,
// invalid ids), and returns non-zero on any wrong result; the sanitizers abort on a race, an invalid
// access or undefined behaviour.
#include <cmath>
#include <cstdint>
#include <cstdio>

extern "C" {
int z2h_protocol_sim_steps(int world, int steps, int buckets, unsigned int first_epoch);
int z2h_protocol_sim_silent_peer(int world, int budget_ms, int* out);
int z2h_protocol_sim_last_one_out(int n, int groups);
int32_t mg_leaf(double value);
int32_t mg_op(int32_t op, int32_t a, int32_t b, double aux);
int32_t mg_affine(int32_t n, const int32_t* w, const int32_t* x, int32_t b);
double mg_get_data(int32_t id);
double mg_get_grad(int32_t id);
void mg_release(int32_t id);
int32_t mg_backward(int32_t root);
int32_t mg_live_nodes();
}

#define CHECK(cond)                                                      \
  do {                                                                   \
    if (!(cond)) {                                                       \
      std::fprintf(stderr, "FAILED line %d: %s\n", __LINE__, #cond);     \
      return 1;                                                          \
    }                                                                    \
  } while (0)

int main() {
  // protocol: 8 ranks, 6 steps of 5 bucket barriers + the norm exchange, starting 3 steps before the wrap
  CHECK(z2h_protocol_sim_steps(8, 6, 5, 0xFFFFFFFDu) == 0);
  CHECK(z2h_protocol_sim_steps(2, 3, 64, 0u) == 0);
  int out[4 * 4] = {};
  CHECK(z2h_protocol_sim_silent_peer(4, 150, out) == 0);
  for (int r = 0; r < 3; ++r) {
    CHECK(out[4 * r + 0] == 0);  // step 1 timed out, as it must
    CHECK(out[4 * r + 1] == 5);  // with the peer-timeout status
    CHECK(out[4 * r + 2] == 1);  // step 2 completed, and not on the late signal of step 1
  }
  CHECK(z2h_protocol_sim_last_one_out(8, 50) == 50);

  // micrograd: y = tanh(w0 x0 + w1 x1 + b) twice over, with node slots released and reused in between
  for (int round = 0; round < 3; ++round) {
    const int before = mg_live_nodes();
    int32_t w[2] = {mg_leaf(0.5), mg_leaf(-0.25)}, x[2] = {mg_leaf(2.0), mg_leaf(4.0)};
    const int32_t b = mg_leaf(0.1);
    const int32_t z = mg_affine(2, w, x, b);
    const int32_t y = mg_op(4 /* tanh */, z, -1, 0.0);
    CHECK(z >= 0 && y >= 0);
    CHECK(std::fabs(mg_get_data(z) - 0.1) < 1e-12);
    CHECK(mg_backward(y) >= 0);
    const double t = std::tanh(0.1), dz = 1.0 - t * t;
    CHECK(std::fabs(mg_get_grad(w[0]) - dz * 2.0) < 1e-12);
    CHECK(std::fabs(mg_get_grad(x[1]) - dz * -0.25) < 1e-12);
    CHECK(std::fabs(mg_get_grad(b) - dz) < 1e-12);
    const int32_t ids[] = {y, z, b, x[1], x[0], w[1], w[0]};
    for (int32_t id : ids) mg_release(id);
    CHECK(mg_live_nodes() == before);
    CHECK(std::isnan(mg_get_data(y)));         // a released id reads as NaN, it does not fault
    CHECK(mg_op(1 /* add */, y, z, 0.0) < 0);  // and cannot be used as an operand
    CHECK(mg_backward(-7) < 0);
  }
  std::puts("host sanitize OK");
  return 0;
}
