// Scalar reverse-mode autograd engine (host C++), the native core behind
// zero_to_hero_b200.micrograd.Value.
//
// Nodes live in an arena indexed by integer handles; a node stores its value, gradient, op code
// and up to two child handles. backward(root) does an iterative post-order walk of the
// sub-graph under root (explicit stack, visit stamps instead of a set) and then sweeps it in
// reverse, adding into the children's gradients, which is exactly the behaviour of the
// reference's Python engine (nn/micrograd/value.py:17-34: gradients accumulate with +=, the
// root's gradient is set to 1). Handles are recycled when the owning Python object dies.
//
// Besides the unary / binary scalar ops there is one n-ary node, kAffine: b + sum_i w_i * x_i in
// a single node (children w_0..w_{n-1}, x_0..x_{n-1}, b). A neuron of the MLP classes
// (zero_to_hero_b200/micrograd/nn.py) is then two nodes (affine, tanh) instead of 2n+1, which
// is what makes a training epoch cheap: the graph walk and the Python object count shrink by
// the fan-in.
#include <cmath>
#include <cstdint>
#include <mutex>
#include <vector>

namespace {

enum Op : int32_t {
  kLeaf = 0, kAdd, kMul, kPow, kTanh, kRelu, kSigmoid, kExp, kLog, kAbs, kDiv, kAffine,
};

struct Node {
  double data = 0.0, grad = 0.0, aux = 0.0;  // aux: exponent of kPow
  int32_t op = kLeaf;
  int32_t a = -1, b = -1;
  uint32_t stamp = 0;
  bool alive = false;
};

std::vector<Node> g_nodes;
std::vector<std::vector<int32_t>> g_kids;  // children of n-ary nodes, indexed like g_nodes
std::vector<int32_t> g_free;
uint32_t g_stamp = 0;
std::mutex g_mutex;

int32_t alloc_node() {
  int32_t id;
  if (!g_free.empty()) {
    id = g_free.back();
    g_free.pop_back();
    g_nodes[id] = Node();
    g_kids[id].clear();
  } else {
    id = (int32_t)g_nodes.size();
    g_nodes.emplace_back();
    g_kids.emplace_back();
  }
  g_nodes[id].alive = true;
  return id;
}

inline bool valid(int32_t id) { return id >= 0 && id < (int32_t)g_nodes.size() && g_nodes[id].alive; }

void backprop_one(Node& n) {
  const double g = n.grad;
  switch (n.op) {
    case kAdd:
      g_nodes[n.a].grad += g;
      g_nodes[n.b].grad += g;
      break;
    case kMul: {
      const double da = g_nodes[n.a].data, db = g_nodes[n.b].data;
      g_nodes[n.a].grad += g * db;
      g_nodes[n.b].grad += g * da;
      break;
    }
    case kDiv: {
      const double da = g_nodes[n.a].data, db = g_nodes[n.b].data;
      g_nodes[n.a].grad += g / db;
      g_nodes[n.b].grad += g * (-da / (db * db));
      break;
    }
    case kPow: g_nodes[n.a].grad += g * n.aux * std::pow(g_nodes[n.a].data, n.aux - 1.0); break;
    case kTanh: g_nodes[n.a].grad += g * (1.0 - n.data * n.data); break;
    case kRelu: g_nodes[n.a].grad += g * (n.data > 0.0 ? 1.0 : 0.0); break;
    case kSigmoid: g_nodes[n.a].grad += g * n.data * (1.0 - n.data); break;
    case kExp: g_nodes[n.a].grad += g * n.data; break;
    case kLog: g_nodes[n.a].grad += g / g_nodes[n.a].data; break;
    case kAbs: {
      const double x = g_nodes[n.a].data;
      g_nodes[n.a].grad += g * (x > 0.0 ? 1.0 : (x < 0.0 ? -1.0 : 0.0));
      break;
    }
    case kAffine: {
      const std::vector<int32_t>& k = g_kids[&n - g_nodes.data()];
      const size_t fan_in = (k.size() - 1) / 2;
      for (size_t i = 0; i < fan_in; ++i) {
        Node& w = g_nodes[k[i]];
        Node& x = g_nodes[k[fan_in + i]];
        const double wd = w.data, xd = x.data;  // w and x may be the same node
        w.grad += g * xd;
        x.grad += g * wd;
      }
      g_nodes[k.back()].grad += g;
      break;
    }
    default: break;
  }
}

}  // namespace

extern "C" {

int32_t mg_leaf(double value) {
  std::lock_guard<std::mutex> lock(g_mutex);
  const int32_t id = alloc_node();
  g_nodes[id].data = value;
  return id;
}

// op: 1 add, 2 mul, 10 div (binary); 3 pow (aux = exponent); 4..9 unary
int32_t mg_op(int32_t op, int32_t a, int32_t b, double aux) {
  std::lock_guard<std::mutex> lock(g_mutex);
  const bool binary = (op == kAdd || op == kMul || op == kDiv);
  if (!valid(a) || (binary && !valid(b))) return -1;
  const double x = g_nodes[a].data;
  double out = 0.0;
  switch (op) {
    case kAdd: out = x + g_nodes[b].data; break;
    case kMul: out = x * g_nodes[b].data; break;
    case kDiv: out = x / g_nodes[b].data; break;
    case kPow: out = std::pow(x, aux); break;
    case kTanh: out = std::tanh(x); break;
    case kRelu: out = x > 0.0 ? x : 0.0; break;
    case kSigmoid: out = 1.0 / (1.0 + std::exp(-x)); break;
    case kExp: out = std::exp(x); break;
    case kLog: out = std::log(x); break;
    case kAbs: out = std::fabs(x); break;
    default: return -1;
  }
  const int32_t id = alloc_node();
  Node& n = g_nodes[id];
  n.data = out;
  n.op = op;
  n.a = a;
  n.b = binary ? b : -1;
  n.aux = aux;
  return id;
}

// b + sum_i w[i] * x[i] as one node (products added in index order, starting from b).
int32_t mg_affine(int32_t n, const int32_t* w, const int32_t* x, int32_t b) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (n < 0 || !valid(b)) return -1;
  for (int32_t i = 0; i < n; ++i)
    if (!valid(w[i]) || !valid(x[i])) return -1;
  double out = g_nodes[b].data;
  for (int32_t i = 0; i < n; ++i) out += g_nodes[w[i]].data * g_nodes[x[i]].data;
  const int32_t id = alloc_node();
  g_nodes[id].data = out;
  g_nodes[id].op = kAffine;
  std::vector<int32_t>& k = g_kids[id];
  k.reserve(2 * (size_t)n + 1);
  k.insert(k.end(), w, w + n);
  k.insert(k.end(), x, x + n);
  k.push_back(b);
  return id;
}

double mg_get_data(int32_t id) { return valid(id) ? g_nodes[id].data : NAN; }
double mg_get_grad(int32_t id) { return valid(id) ? g_nodes[id].grad : NAN; }
void mg_set_data(int32_t id, double v) { if (valid(id)) g_nodes[id].data = v; }
void mg_set_grad(int32_t id, double v) { if (valid(id)) g_nodes[id].grad = v; }

void mg_release(int32_t id) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (valid(id)) {
    g_nodes[id].alive = false;
    g_free.push_back(id);
  }
}

// Returns the number of nodes visited, or -1 for a bad handle.
int32_t mg_backward(int32_t root) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!valid(root)) return -1;
  ++g_stamp;
  std::vector<int32_t> order, stack;
  stack.push_back(root);
  // stamp values: g_stamp marks "finished"; a node is expanded at most once per child scan
  while (!stack.empty()) {
    const int32_t id = stack.back();
    Node& n = g_nodes[id];
    if (n.stamp == g_stamp) {  // reached again through another parent
      stack.pop_back();
      continue;
    }
    bool ready = true;
    const int32_t pair[2] = {n.a, n.b};
    const bool nary = n.op == kAffine;
    const int32_t* kids = nary ? g_kids[id].data() : pair;
    const size_t n_kids = nary ? g_kids[id].size() : 2;
    for (size_t k = 0; k < n_kids; ++k) {
      const int32_t c = kids[k];
      if (c >= 0 && g_nodes[c].stamp != g_stamp) {
        ready = false;
        stack.push_back(c);
      }
    }
    if (ready) {
      n.stamp = g_stamp;
      order.push_back(id);
      stack.pop_back();
    }
  }
  g_nodes[root].grad = 1.0;
  for (auto it = order.rbegin(); it != order.rend(); ++it) backprop_one(g_nodes[*it]);
  return (int32_t)order.size();
}

int32_t mg_live_nodes() {
  std::lock_guard<std::mutex> lock(g_mutex);
  return (int32_t)(g_nodes.size() - g_free.size());
}

}
