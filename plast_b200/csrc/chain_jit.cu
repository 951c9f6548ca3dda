// Run-time compilation of fused elementwise chains.
//
// plast_b200_chain_forward receives a straight-line program of elementwise steps. Interpreting it
// inside a kernel keeps the result exact but indexes a per-thread register file dynamically, which
// lands in local memory and costs a multiple of the HBM time. Here the program is turned into a
// functor in CUDA C++ (one `const float rK = ...;` per step, every step still rounded on its own:
// NVRTC gets --fmad=false), compiled by NVRTC for sm_100a together with the very same ew_kernel
// template the ahead-of-time build uses (ew_kernel_device.cuh is embedded as text), and launched
// through the driver API. Compiled kernels are cached per (program structure, inputs, vector
// width, index width, 1-D); scalar constants travel as kernel arguments, so a chain that differs
// only in its constants reuses the binary. This is the role the reference's README assigns to its
// NVRTC JIT ("in development", README.md:90,188).
//
// libnvrtc and libcuda are opened with dlopen on first use; when either is missing, or a compile
// fails, the caller falls back to the in-kernel interpreter (still a GPU kernel of this library).
#include "ew_engine.cuh"

#include <dlfcn.h>
#include <string.h>
#include <mutex>
#include <string>
#include <unordered_map>

namespace pb {

static const char *kDeviceSource =
#include "ew_kernel_device_src.inc"
    ;

struct ChainProgramView { // mirrors ChainProgram of chain.cu (kept POD so both files agree)
  int n_inputs, n_steps;
  const unsigned char *opcode, *a, *b;
  const float *fval;
  // bit i set: input i is one element whatever the output index (a 0-dim constant such as the 1.0
  // of `1.0 + x`). Such inputs are read once per thread through a pointer in the functor instead
  // of occupying an operand slot of the kernel (registers and a load per element).
  unsigned scalar_mask;
  // wrt < 0: the forward functor. wrt >= 0: the backward functor for input `wrt`: operand 0 of the
  // kernel is the upstream gradient, the chain's tensor inputs follow, and with `accumulate` the
  // last operand is the input's current gradient, which the returned value replaces.
  int wrt;
  bool accumulate;
};
// Operands of the generated kernel: [upstream gradient] + tensor inputs + [current gradient].
static int tensor_inputs(const ChainProgramView &p) {
  int n = 0;
  for (int i = 0; i < p.n_inputs; ++i) n += !((p.scalar_mask >> i) & 1u);
  if (p.wrt >= 0) n += 1 + (p.accumulate ? 1 : 0);
  return n;
}

// ---- minimal NVRTC / driver API surface, resolved at run time -------------------------------------
typedef int nvrtcResult;
typedef struct _nvrtcProgram *nvrtcProgram;
typedef int CUresult;
typedef struct CUmod_st *CUmodule;
typedef struct CUfunc_st *CUfunction;
typedef struct CUstream_st *CUstream;

struct Api {
  bool ok = false;      // compiler and driver both available
  bool rtc_ok = false;  // compiler available (enough to check that a program compiles)
  nvrtcResult (*CreateProgram)(nvrtcProgram *, const char *, const char *, int, const char *const *,
                               const char *const *) = nullptr;
  nvrtcResult (*DestroyProgram)(nvrtcProgram *) = nullptr;
  nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char *const *) = nullptr;
  nvrtcResult (*AddNameExpression)(nvrtcProgram, const char *) = nullptr;
  nvrtcResult (*GetLoweredName)(nvrtcProgram, const char *, const char **) = nullptr;
  nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t *) = nullptr;
  nvrtcResult (*GetCUBIN)(nvrtcProgram, char *) = nullptr;
  nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t *) = nullptr;
  nvrtcResult (*GetProgramLog)(nvrtcProgram, char *) = nullptr;
  CUresult (*ModuleLoadData)(CUmodule *, const void *) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction *, CUmodule, const char *) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                           unsigned, CUstream, void **, void **) = nullptr;
};

template <class Fn> bool resolve(void *lib, const char *name, Fn *out) {
  *out = reinterpret_cast<Fn>(dlsym(lib, name));
  return *out != nullptr;
}

Api &api() {
  static Api a = [] {
    Api r;
    void *rtc = nullptr;
    for (const char *n : {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12"}) {
      rtc = dlopen(n, RTLD_NOW | RTLD_LOCAL);
      if (rtc) break;
    }
    void *drv = dlopen("libcuda.so.1", RTLD_NOW | RTLD_LOCAL);
    if (!rtc) return r;
    bool ok = resolve(rtc, "nvrtcCreateProgram", &r.CreateProgram) &&
              resolve(rtc, "nvrtcDestroyProgram", &r.DestroyProgram) &&
              resolve(rtc, "nvrtcCompileProgram", &r.CompileProgram) &&
              resolve(rtc, "nvrtcAddNameExpression", &r.AddNameExpression) &&
              resolve(rtc, "nvrtcGetLoweredName", &r.GetLoweredName) &&
              resolve(rtc, "nvrtcGetCUBINSize", &r.GetCUBINSize) &&
              resolve(rtc, "nvrtcGetCUBIN", &r.GetCUBIN) &&
              resolve(rtc, "nvrtcGetProgramLogSize", &r.GetProgramLogSize) &&
              resolve(rtc, "nvrtcGetProgramLog", &r.GetProgramLog);
    r.rtc_ok = ok;
    r.ok = ok && drv && resolve(drv, "cuModuleLoadData", &r.ModuleLoadData) &&
           resolve(drv, "cuModuleGetFunction", &r.ModuleGetFunction) &&
           resolve(drv, "cuLaunchKernel", &r.LaunchKernel);
    return r;
  }();
  return a;
}

// ---- source generation --------------------------------------------------------------------------------
const char *step_expr(int opcode) {
  switch (opcode) {
  case PLAST_CHAIN_ADD: return "A + B";
  case PLAST_CHAIN_SUB: return "A - B";
  case PLAST_CHAIN_MUL: return "A * B";
  case PLAST_CHAIN_DIV: return "A / B";
  case PLAST_CHAIN_NEG: return "-A";
  case PLAST_CHAIN_ABS: return "fabsf(A)";
  case PLAST_CHAIN_EXP: return "expf(A)";
  case PLAST_CHAIN_LOG: return "logf(A)";
  case PLAST_CHAIN_SIN: return "sinf(A)";
  case PLAST_CHAIN_COS: return "cosf(A)";
  case PLAST_CHAIN_TAN: return "(float)tan((double)A)";
  case PLAST_CHAIN_LEAKY_RELU: return "(A > 0.0f ? A : A * C)";
  case PLAST_CHAIN_ADD_SCALAR: return "A + C";
  case PLAST_CHAIN_RSUB_SCALAR: return "C - A";
  case PLAST_CHAIN_MUL_SCALAR: return "A * C";
  default: return "C / A"; // PLAST_CHAIN_RDIV_SCALAR
  }
}

// Gradient statements of one step, in the order the standalone backward kernels apply them
// (first operand, then second; functors.cuh): GA / GB are the adjoint registers of the operands,
// G the adjoint of the step's result, R the step's forward value.
const char *step_backward(int opcode) {
  switch (opcode) {
  case PLAST_CHAIN_ADD: return "GA = GA + G; GB = GB + G;";
  case PLAST_CHAIN_SUB: return "GA = GA + G; GB = GB + (-G);";
  case PLAST_CHAIN_MUL: return "GA = GA + G * B; GB = GB + G * A;";
  case PLAST_CHAIN_DIV: return "GA = GA + G / B; GB = GB + (-G * A / (B * B));";
  case PLAST_CHAIN_NEG: return "GA = GA - G;";
  case PLAST_CHAIN_ABS: return "GA = GA + G * (A > 0.0f ? 1.0f : (A < 0.0f ? -1.0f : 0.0f));";
  case PLAST_CHAIN_EXP: return "GA = GA + G * R;";
  case PLAST_CHAIN_LOG: return "GA = GA + G * (1.0f / A);";
  case PLAST_CHAIN_SIN: return "GA = GA + G * cosf(A);";
  case PLAST_CHAIN_COS: return "GA = GA + G * (-sinf(A));";
  case PLAST_CHAIN_TAN: return "GA = GA + G * (1.0f + R * R);";
  case PLAST_CHAIN_LEAKY_RELU: return "GA = GA + G * (A > 0.0f ? 1.0f : C);";
  case PLAST_CHAIN_ADD_SCALAR: return "GA = GA + G;";
  case PLAST_CHAIN_RSUB_SCALAR: return "GA = GA + (-G);";
  case PLAST_CHAIN_MUL_SCALAR: return "GA = GA + G * C;";
  default: return "GA = GA + (-G * C / (A * A));"; // PLAST_CHAIN_RDIV_SCALAR
  }
}

std::string functor_source(const ChainProgramView &p) {
  std::string s = "namespace pb {\nstruct JitF {\n  float c[" + std::to_string(PLAST_CHAIN_MAX_STEPS) +
                  "];\n  const float *sp[" + std::to_string(PLAST_CHAIN_MAX_INPUTS) +
                  "];\n  __device__ __forceinline__ float operator()(const float *x) const {\n";
  const bool backward = p.wrt >= 0;
  if (backward) s += "    const float g = x[0];\n";
  for (int i = 0, slot = backward ? 1 : 0, sc = 0; i < p.n_inputs; ++i) {
    if ((p.scalar_mask >> i) & 1u)
      s += "    const float r" + std::to_string(i) + " = __ldg(sp[" + std::to_string(sc++) + "]);\n";
    else
      s += "    const float r" + std::to_string(i) + " = x[" + std::to_string(slot++) + "];\n";
  }
  for (int k = 0; k < p.n_steps; ++k) {
    std::string e = step_expr(p.opcode[k]);
    auto sub = [&](const std::string &from, const std::string &to) {
      for (size_t pos = 0; (pos = e.find(from, pos)) != std::string::npos; pos += to.size())
        e.replace(pos, from.size(), to);
    };
    // single capital letters never occur in the function names above except as placeholders
    sub("A", "r" + std::to_string(p.a[k]));
    sub("B", "r" + std::to_string(p.b[k]));
    sub("C", "c[" + std::to_string(k) + "]");
    s += "    const float r" + std::to_string(p.n_inputs + k) + " = " + e + ";\n";
  }
  if (!backward) {
    s += "    return r" + std::to_string(p.n_inputs + p.n_steps - 1) + ";\n  }\n};\n} // namespace pb\n";
    return s;
  }
  // Reverse sweep. Every adjoint starts at zero and receives its contributions in the order the
  // node-by-node backward applies them (later nodes first), each rounded on its own, so the
  // result equals the unfused backward bit for bit; the wanted input's adjoint starts from its
  // current gradient when that is an operand. Adjoints nobody returns are dead code.
  const int n_regs = p.n_inputs + p.n_steps;
  for (int r = 0; r < n_regs; ++r) {
    std::string init = "0.0f";
    if (r == p.wrt && p.accumulate) init = "x[" + std::to_string(tensor_inputs(p) - 1) + "]";
    if (r == n_regs - 1) init = "g";
    s += "    float a" + std::to_string(r) + " = " + init + ";\n";
  }
  for (int k = p.n_steps - 1; k >= 0; --k) {
    std::string e = step_backward(p.opcode[k]);
    auto sub = [&](const std::string &from, const std::string &to) {
      for (size_t pos = 0; (pos = e.find(from, pos)) != std::string::npos; pos += to.size())
        e.replace(pos, from.size(), to);
    };
    // two-letter placeholders first; single capitals never occur in the function names used
    sub("GA", "a" + std::to_string(p.a[k]));
    sub("GB", "a" + std::to_string(p.b[k]));
    sub("G", "a" + std::to_string(p.n_inputs + k));
    sub("A", "r" + std::to_string(p.a[k]));
    sub("B", "r" + std::to_string(p.b[k]));
    sub("R", "r" + std::to_string(p.n_inputs + k));
    sub("C", "c[" + std::to_string(k) + "]");
    s += "    " + e + "\n";
  }
  s += "    return a" + std::to_string(p.wrt) + ";\n  }\n};\n} // namespace pb\n";
  return s;
}

std::string structure_key(const ChainProgramView &p) {
  std::string k = std::to_string(p.n_inputs) + "/" + std::to_string(p.scalar_mask) + "/" +
                  std::to_string(p.wrt) + (p.accumulate ? "+" : "") + ":";
  for (int i = 0; i < p.n_steps; ++i)
    k += std::to_string(p.opcode[i]) + "," + std::to_string(p.a[i]) + "," + std::to_string(p.b[i]) + ";";
  return k;
}

std::string instance_name(const ChainProgramView &p, int vec, bool idx64, bool one_d, unsigned cmask = 0) {
  return "pb::ew_kernel<pb::JitF, " + std::to_string(tensor_inputs(p)) + ", " + std::to_string(vec) + ", " +
         (idx64 ? "unsigned long long" : "unsigned int") + ", " + (one_d ? "true" : "false") + ", " +
         std::to_string(cmask) + "u>";
}
std::string program_source(const ChainProgramView &p, const std::string &inst, bool idx64) {
  const char *idx = idx64 ? "unsigned long long" : "unsigned int";
  return std::string(kDeviceSource) + "\n" + functor_source(p) + "\ntemplate __global__ void " + inst +
         "(pb::JitF, float *, pb::InPtrs<" + std::to_string(tensor_inputs(p)) + ">, pb::OffsetCalc<" +
         std::to_string(tensor_inputs(p) + 1) + ", " + idx + ">, " + idx + ", unsigned int);\n";
}

std::mutex g_mutex;
std::unordered_map<std::string, CUfunction> g_cache; // nullptr = compile failed, do not retry

CUfunction get_kernel(const ChainProgramView &p, int vec, bool idx64, bool one_d, unsigned cmask) {
  Api &a = api();
  if (!a.ok) return nullptr;
  const std::string inst = instance_name(p, vec, idx64, one_d, cmask);
  const std::string key = structure_key(p) + inst;
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = g_cache.find(key);
  if (it != g_cache.end()) return it->second;
  CUfunction fn = nullptr;
  const std::string src = program_source(p, inst, idx64);
  nvrtcProgram prog = nullptr;
  if (a.CreateProgram(&prog, src.c_str(), "plast_chain.cu", 0, nullptr, nullptr) == 0) {
    a.AddNameExpression(prog, inst.c_str());
    const char *opts[] = {"--gpu-architecture=sm_100a", "--fmad=false", "--std=c++17"};
    const nvrtcResult rc = a.CompileProgram(prog, 3, opts);
    if (rc == 0) {
      const char *lowered = nullptr;
      size_t size = 0;
      if (a.GetLoweredName(prog, inst.c_str(), &lowered) == 0 && lowered &&
          a.GetCUBINSize(prog, &size) == 0 && size > 0) {
        std::string cubin(size, '\0');
        CUmodule mod = nullptr;
        if (a.GetCUBIN(prog, &cubin[0]) == 0 && a.ModuleLoadData(&mod, cubin.data()) == 0)
          if (a.ModuleGetFunction(&fn, mod, lowered) != 0) fn = nullptr;
      }
    } else {
      size_t n = 0;
      a.GetProgramLogSize(prog, &n);
      std::string log(n + 1, '\0');
      if (n) a.GetProgramLog(prog, &log[0]);
      fprintf(stderr, "plast: chain JIT compile failed (%d), using the interpreter:\n%s\n", rc, log.c_str());
    }
    a.DestroyProgram(&prog);
  }
  g_cache[key] = fn;
  return fn;
}

struct JitFHost {
  float c[PLAST_CHAIN_MAX_STEPS];
  const float *sp[PLAST_CHAIN_MAX_INPUTS];
};

template <int NIN, typename index_t>
bool launch_variant(CUfunction fn, const IterPlan &plan, float *out, const float *const *ins,
                    const JitFHost &f, int vec, u64 n_items, uint32_t vec_mask, unsigned blocks) {
  InPtrs<NIN> ip;
  for (int a = 0; a < NIN; ++a) ip.p[a] = ins[a];
  OffsetCalc<NIN + 1, index_t> oc;
  fill_offset_calc(&oc, plan, vec);
  index_t n = (index_t)n_items;
  JitFHost fcopy = f;
  void *args[] = {&fcopy, &out, &ip, &oc, &n, &vec_mask};
  return api().LaunchKernel(fn, blocks, 1, 1, kEwThreads, 1, 1, 0, (CUstream)stream(), args, nullptr) == 0;
}

template <int NIN>
bool launch_one(const ChainProgramView &p, const IterPlan &plan, float *out, const float *const *ins,
                const JitFHost &f) {
  if (plan.numel == 0) return true;
  const void *ptrs[NIN + 1];
  ptrs[0] = out;
  for (int a = 0; a < NIN; ++a) ptrs[a + 1] = ins[a];
  u64 n_items = 0;
  uint32_t vec_mask = 0;
  const EwChoice c = choose_ew(plan, ptrs, NIN + 1, &n_items, &vec_mask);
  const u64 per_block = (u64)kEwThreads * kEwUnroll;
  const u64 blocks = (n_items + per_block - 1) / per_block;
  if (blocks > 0x7fffffffull) return false;
  // same compile-time operand masks as the ahead-of-time engine
  const unsigned cmask = (NIN >= 2 && c.vec == 4 && !c.idx64 && (vec_mask == 1u || vec_mask == 2u)) ? vec_mask : 0u;
  CUfunction fn = get_kernel(p, c.vec, c.idx64, c.one_d, cmask);
  if (!fn) return false;
  const bool ok = c.idx64 ? launch_variant<NIN, uint64_t>(fn, plan, out, ins, f, c.vec, n_items, vec_mask, (unsigned)blocks)
                          : launch_variant<NIN, uint32_t>(fn, plan, out, ins, f, c.vec, n_items, vec_mask, (unsigned)blocks);
  if (ok) count_launch();
  return ok;
}

template <int NIN>
bool launch_plan(const ChainProgramView &p, const IterPlan &plan, float *out, const float *const *ins,
                 const JitFHost &f) {
  // same body + tail split as launch_ew for 1-D plans of odd length
  if (plan.ndim == 1 && plan.size[0] >= 8 && (plan.size[0] & 3) != 0 && plan.stride[0][0] == 1) {
    bool ok = true;
    for (int a = 1; a <= NIN; ++a) ok = ok && plan.stride[a][0] <= 1;
    if (ok) {
      const u64 body_n = plan.size[0] & ~(u64)3;
      IterPlan body = plan, tail = plan;
      body.size[0] = body_n;
      body.numel = body_n;
      tail.size[0] = plan.size[0] - body_n;
      tail.numel = tail.size[0];
      const float *tins[NIN];
      for (int a = 0; a <= NIN; ++a) {
        body.max_offset[a] = (body_n - 1) * plan.stride[a][0];
        tail.max_offset[a] = (tail.size[0] - 1) * plan.stride[a][0];
        if (a > 0) tins[a - 1] = ins[a - 1] + body_n * plan.stride[a][0];
      }
      return launch_one<NIN>(p, body, out, ins, f) && launch_one<NIN>(p, tail, out + body_n, tins, f);
    }
  }
  return launch_one<NIN>(p, plan, out, ins, f);
}

// Returns false when the chain could not be compiled or launched this way; nothing has been
// launched in that case (a failed tail after a launched body is reported as an error instead).
//
// Operand layout of `plan` / `ins`: forward (p.wrt < 0): the chain's inputs. Backward: the upstream
// gradient, then the chain's inputs, then (p.accumulate) the current gradient of input p.wrt.
static bool jit_disabled_by_env() {
  static const bool disabled = [] {
    const char *e = getenv("PLAST_B200_CHAIN_JIT");
    return e && e[0] == '0';
  }();
  return disabled;
}

bool launch_chain_jit(const ChainProgramView &p, const IterPlan &plan, float *out, const float *const *ins) {
  if (jit_disabled_by_env() || !api().ok) return false;
  JitFHost f = {};
  for (int k = 0; k < p.n_steps; ++k) f.c[k] = p.fval[k];
  // Inputs the plan never advances are constants: hand them to the functor as pointers and plan
  // the launch over the remaining operands only (at least one stays, so the kernel has an operand).
  ChainProgramView q = p;
  q.scalar_mask = 0;
  IterPlan lean = plan;
  constexpr int kMaxOperands = PLAST_CHAIN_MAX_INPUTS + 2;
  const float *tensor_ins[kMaxOperands] = {};
  int n_tensor = 0, n_scalar = 0;
  auto keep = [&](int arg) { // plan argument `arg` (>= 1) stays a kernel operand
    for (int d = 0; d < MAX_NDIM; ++d) lean.stride[n_tensor + 1][d] = plan.stride[arg][d];
    lean.max_offset[n_tensor + 1] = plan.max_offset[arg];
    tensor_ins[n_tensor++] = ins[arg - 1];
  };
  const int first = p.wrt >= 0 ? 1 : 0; // operand index of the chain's input 0
  if (p.wrt >= 0) keep(1);
  for (int a = 0; a < p.n_inputs; ++a) {
    bool moves = false;
    for (int d = 0; d < plan.ndim; ++d) moves = moves || plan.stride[first + a + 1][d] != 0;
    if (!moves && !(n_tensor == 0 && a == p.n_inputs - 1)) {
      q.scalar_mask |= 1u << a;
      f.sp[n_scalar++] = ins[first + a];
      continue;
    }
    keep(first + a + 1);
  }
  if (p.wrt >= 0 && p.accumulate) keep(first + p.n_inputs + 1);
  lean.nargs = n_tensor + 1;
  switch (n_tensor) {
  case 1: return launch_plan<1>(q, lean, out, tensor_ins, f);
  case 2: return launch_plan<2>(q, lean, out, tensor_ins, f);
  case 3: return launch_plan<3>(q, lean, out, tensor_ins, f);
  case 4: return launch_plan<4>(q, lean, out, tensor_ins, f);
  case 5: return launch_plan<5>(q, lean, out, tensor_ins, f);
  case 6: return launch_plan<6>(q, lean, out, tensor_ins, f);
  case 7: return launch_plan<7>(q, lean, out, tensor_ins, f);
  case 8: return launch_plan<8>(q, lean, out, tensor_ins, f);
  case 9: return launch_plan<9>(q, lean, out, tensor_ins, f);
  case 10: return launch_plan<10>(q, lean, out, tensor_ins, f);
  default: return false;
  }
}

bool chain_jit_available() { return !jit_disabled_by_env() && api().ok; }

} // namespace pb

// ---- test hooks (declared in include/plast_b200.h; need no GPU) ------------------------------------------
static bool view_of(const PlastChainStep *steps, int n_steps, int n_inputs, unsigned scalar_mask,
                    unsigned char *op, unsigned char *a, unsigned char *b, float *f, pb::ChainProgramView *v) {
  if (!steps || n_inputs < 1 || n_inputs > PLAST_CHAIN_MAX_INPUTS || n_steps < 1 || n_steps > PLAST_CHAIN_MAX_STEPS)
    return false;
  if (scalar_mask >> n_inputs || scalar_mask == (1u << n_inputs) - 1u) return false; // one operand must stay
  for (int s = 0; s < n_steps; ++s) {
    const bool binary = steps[s].opcode <= PLAST_CHAIN_DIV;
    if (steps[s].opcode < 0 || steps[s].opcode > PLAST_CHAIN_RDIV_SCALAR || steps[s].a < 0 ||
        steps[s].a >= n_inputs + s || (binary && (steps[s].b < 0 || steps[s].b >= n_inputs + s)))
      return false;
    op[s] = (unsigned char)steps[s].opcode;
    a[s] = (unsigned char)steps[s].a;
    b[s] = (unsigned char)(binary ? steps[s].b : steps[s].a);
    f[s] = steps[s].fval;
  }
  *v = pb::ChainProgramView{n_inputs, n_steps, op, a, b, f, scalar_mask, -1, false};
  return true;
}

extern "C" int plast_b200_chain_source(const PlastChainStep *steps, int n_steps, int n_inputs,
                                       unsigned scalar_mask, char *buf, size_t capacity) {
  unsigned char op[PLAST_CHAIN_MAX_STEPS], a[PLAST_CHAIN_MAX_STEPS], b[PLAST_CHAIN_MAX_STEPS];
  float f[PLAST_CHAIN_MAX_STEPS];
  pb::ChainProgramView v;
  if (!view_of(steps, n_steps, n_inputs, scalar_mask, op, a, b, f, &v)) return -1;
  const std::string src = pb::functor_source(v);
  if (buf && capacity > 0) {
    const size_t n = src.size() < capacity - 1 ? src.size() : capacity - 1;
    memcpy(buf, src.data(), n);
    buf[n] = 0;
  }
  return (int)src.size();
}

extern "C" int plast_b200_chain_backward_source(const PlastChainStep *steps, int n_steps, int n_inputs,
                                                unsigned scalar_mask, int wrt, int accumulate, char *buf,
                                                size_t capacity) {
  unsigned char op[PLAST_CHAIN_MAX_STEPS], a[PLAST_CHAIN_MAX_STEPS], b[PLAST_CHAIN_MAX_STEPS];
  float f[PLAST_CHAIN_MAX_STEPS];
  pb::ChainProgramView v;
  if (!view_of(steps, n_steps, n_inputs, scalar_mask, op, a, b, f, &v) || wrt < 0 || wrt >= n_inputs) return -1;
  v.wrt = wrt;
  v.accumulate = accumulate != 0;
  const std::string src = pb::functor_source(v);
  if (buf && capacity > 0) {
    const size_t n = src.size() < capacity - 1 ? src.size() : capacity - 1;
    memcpy(buf, src.data(), n);
    buf[n] = 0;
  }
  return (int)src.size();
}

extern "C" int plast_b200_chain_jit_available(void) { return pb::chain_jit_available() ? 1 : 0; }

static int try_compile_view(const pb::ChainProgramView &v) {
  pb::Api &api = pb::api();
  if (!api.rtc_ok) return -2;
  const std::string inst = pb::instance_name(v, 4, false, true);
  const std::string src = pb::program_source(v, inst, false);
  pb::nvrtcProgram prog = nullptr;
  if (api.CreateProgram(&prog, src.c_str(), "plast_chain.cu", 0, nullptr, nullptr) != 0) return -3;
  api.AddNameExpression(prog, inst.c_str());
  const char *opts[] = {"--gpu-architecture=sm_100a", "--fmad=false", "--std=c++17"};
  const int rc = api.CompileProgram(prog, 3, opts);
  if (rc != 0) {
    size_t n = 0;
    api.GetProgramLogSize(prog, &n);
    std::string log(n + 1, '\0');
    if (n) api.GetProgramLog(prog, &log[0]);
    fprintf(stderr, "%s\n", log.c_str());
  }
  api.DestroyProgram(&prog);
  return rc;
}

extern "C" int plast_b200_chain_try_compile(const PlastChainStep *steps, int n_steps, int n_inputs,
                                            unsigned scalar_mask) {
  unsigned char op[PLAST_CHAIN_MAX_STEPS], a[PLAST_CHAIN_MAX_STEPS], b[PLAST_CHAIN_MAX_STEPS];
  float f[PLAST_CHAIN_MAX_STEPS];
  pb::ChainProgramView v;
  if (!view_of(steps, n_steps, n_inputs, scalar_mask, op, a, b, f, &v)) return -1;
  return try_compile_view(v);
}

extern "C" int plast_b200_chain_backward_try_compile(const PlastChainStep *steps, int n_steps, int n_inputs,
                                                     unsigned scalar_mask, int wrt, int accumulate) {
  unsigned char op[PLAST_CHAIN_MAX_STEPS], a[PLAST_CHAIN_MAX_STEPS], b[PLAST_CHAIN_MAX_STEPS];
  float f[PLAST_CHAIN_MAX_STEPS];
  pb::ChainProgramView v;
  if (!view_of(steps, n_steps, n_inputs, scalar_mask, op, a, b, f, &v) || wrt < 0 || wrt >= n_inputs) return -1;
  v.wrt = wrt;
  v.accumulate = accumulate != 0;
  return try_compile_view(v);
}
