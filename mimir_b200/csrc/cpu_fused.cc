// Fused elementwise programs on the host (reference: internal/sched/fuse.go:200-362: chains of
// elementwise ops become ONE kernel of up to 256 instructions over up to 16 inputs, so the
// intermediate values never go to memory).
//
// A program is a list of instructions over registers.  It runs block by block (512 values): the
// block of every input is read once, every instruction runs over the block with its operands in
// cache, and only the result block is written.  Blocks are handed to the worker pool.  Arithmetic is
// IEEE float32 exactly as the single ops would compute it; exp / log / tanh / sin / cos / erf / log1p /
// expm1 come from glibc's vector math library (libmvec, at most 4 ulp) on AVX2 machines and from
// libm otherwise.
//
// Instruction: {op, dst, a, b} with registers 0 .. n_in-1 = inputs, then temporaries; an operand
// >= kConstBase names constant (operand - kConstBase).  Inputs are float32 arrays of n values, or
// single values (scalar flag) that are broadcast.
#include <cmath>
#include <cstring>

#include "cpu_pool.h"

#define MIMIR_CPU_API extern "C" __attribute__((visibility("default")))

extern "C" {
__m256 _ZGVdN8v_expf(__m256);
__m256 _ZGVdN8v_logf(__m256);
__m256 _ZGVdN8v_tanhf(__m256);
__m256 _ZGVdN8v_sinf(__m256);
__m256 _ZGVdN8v_cosf(__m256);
__m256 _ZGVdN8v_erff(__m256);
__m256 _ZGVdN8v_log1pf(__m256);
__m256 _ZGVdN8v_expm1f(__m256);
}

namespace {

constexpr int kBlock = 512;
constexpr int kMaxRegs = 96;
constexpr int kConstBase = 1 << 20;

enum Op {
  ADD = 0, SUB, MUL, DIV, MAX, MIN,                       // binary
  NEG = 16, ABS, RELU, SQRT, RSQRT, RECIP, EXP, LOG, TANH, SIGMOID, SILU, GELU_TANH, SIN, COS, ERF, LOG1P, EXPM1,
  SIGN, FLOOR, CEIL, SOFTPLUS,                            // unary
};

#define AVX2 __attribute__((target("avx2,fma")))

AVX2 inline __m256 v_sigmoid(__m256 x) {
  const __m256 one = _mm256_set1_ps(1.f);
  return _mm256_div_ps(one, _mm256_add_ps(one, _ZGVdN8v_expf(_mm256_sub_ps(_mm256_setzero_ps(), x))));
}

// one instruction over one block, AVX2
AVX2 void run_instr_avx2(int op, float* d, const float* a, const float* b) {
  const __m256 zero = _mm256_setzero_ps(), one = _mm256_set1_ps(1.f);
  const __m256 absmask = _mm256_castsi256_ps(_mm256_set1_epi32(0x7fffffff));
  for (int i = 0; i < kBlock; i += 8) {
    const __m256 x = _mm256_loadu_ps(a + i);
    __m256 r;
    switch (op) {
      case ADD: r = _mm256_add_ps(x, _mm256_loadu_ps(b + i)); break;
      case SUB: r = _mm256_sub_ps(x, _mm256_loadu_ps(b + i)); break;
      case MUL: r = _mm256_mul_ps(x, _mm256_loadu_ps(b + i)); break;
      case DIV: r = _mm256_div_ps(x, _mm256_loadu_ps(b + i)); break;
      case MAX: {   // NaN in either operand gives NaN, like torch.maximum
        const __m256 y = _mm256_loadu_ps(b + i);
        r = _mm256_blendv_ps(_mm256_max_ps(x, y), _mm256_add_ps(x, y), _mm256_cmp_ps(x, y, _CMP_UNORD_Q));
        break;
      }
      case MIN: {
        const __m256 y = _mm256_loadu_ps(b + i);
        r = _mm256_blendv_ps(_mm256_min_ps(x, y), _mm256_add_ps(x, y), _mm256_cmp_ps(x, y, _CMP_UNORD_Q));
        break;
      }
      case NEG: r = _mm256_xor_ps(x, _mm256_set1_ps(-0.f)); break;
      case ABS: r = _mm256_and_ps(x, absmask); break;
      case RELU: r = _mm256_blendv_ps(_mm256_max_ps(x, zero), x, _mm256_cmp_ps(x, x, _CMP_UNORD_Q)); break;
      case SQRT: r = _mm256_sqrt_ps(x); break;
      case RSQRT: r = _mm256_div_ps(one, _mm256_sqrt_ps(x)); break;
      case RECIP: r = _mm256_div_ps(one, x); break;
      case EXP: r = _ZGVdN8v_expf(x); break;
      case LOG: r = _ZGVdN8v_logf(x); break;
      case TANH: r = _ZGVdN8v_tanhf(x); break;
      case SIGMOID: r = v_sigmoid(x); break;
      case SILU: r = _mm256_mul_ps(x, v_sigmoid(x)); break;
      case GELU_TANH: {
        const __m256 x3 = _mm256_mul_ps(_mm256_mul_ps(x, x), x);
        const __m256 inner = _mm256_mul_ps(_mm256_set1_ps(0.7978845608028654f), _mm256_fmadd_ps(_mm256_set1_ps(0.044715f), x3, x));
        r = _mm256_mul_ps(_mm256_mul_ps(_mm256_set1_ps(0.5f), x), _mm256_add_ps(one, _ZGVdN8v_tanhf(inner)));
        break;
      }
      case SIN: r = _ZGVdN8v_sinf(x); break;
      case COS: r = _ZGVdN8v_cosf(x); break;
      case ERF: r = _ZGVdN8v_erff(x); break;
      case LOG1P: r = _ZGVdN8v_log1pf(x); break;
      case EXPM1: r = _ZGVdN8v_expm1f(x); break;
      case SIGN: {
        const __m256 pos = _mm256_and_ps(_mm256_cmp_ps(x, zero, _CMP_GT_OQ), one);
        const __m256 neg = _mm256_and_ps(_mm256_cmp_ps(x, zero, _CMP_LT_OQ), one);
        r = _mm256_blendv_ps(_mm256_sub_ps(pos, neg), x, _mm256_cmp_ps(x, x, _CMP_UNORD_Q));
        break;
      }
      case FLOOR: r = _mm256_floor_ps(x); break;
      case CEIL: r = _mm256_ceil_ps(x); break;
      case SOFTPLUS: {   // log(1 + e^x), linear above the threshold of 20 like PyTorch
        const __m256 sp = _ZGVdN8v_log1pf(_ZGVdN8v_expf(_mm256_min_ps(x, _mm256_set1_ps(20.f))));
        r = _mm256_blendv_ps(sp, x, _mm256_cmp_ps(x, _mm256_set1_ps(20.f), _CMP_GT_OQ));
        break;
      }
      default: r = x;
    }
    _mm256_storeu_ps(d + i, r);
  }
}

inline float s_sigmoid(float x) { return 1.f / (1.f + std::exp(-x)); }

// the same, any x86-64
void run_instr_scalar(int op, float* d, const float* a, const float* b) {
  for (int i = 0; i < kBlock; ++i) {
    const float x = a[i];
    float r;
    switch (op) {
      case ADD: r = x + b[i]; break;
      case SUB: r = x - b[i]; break;
      case MUL: r = x * b[i]; break;
      case DIV: r = x / b[i]; break;
      case MAX: r = (x != x || b[i] != b[i]) ? x + b[i] : (x > b[i] ? x : b[i]); break;
      case MIN: r = (x != x || b[i] != b[i]) ? x + b[i] : (x < b[i] ? x : b[i]); break;
      case NEG: r = -x; break;
      case ABS: r = std::fabs(x); break;
      case RELU: r = x != x ? x : (x > 0.f ? x : 0.f); break;
      case SQRT: r = std::sqrt(x); break;
      case RSQRT: r = 1.f / std::sqrt(x); break;
      case RECIP: r = 1.f / x; break;
      case EXP: r = std::exp(x); break;
      case LOG: r = std::log(x); break;
      case TANH: r = std::tanh(x); break;
      case SIGMOID: r = s_sigmoid(x); break;
      case SILU: r = x * s_sigmoid(x); break;
      case GELU_TANH: r = 0.5f * x * (1.f + std::tanh(0.7978845608028654f * (x + 0.044715f * x * x * x))); break;
      case SIN: r = std::sin(x); break;
      case COS: r = std::cos(x); break;
      case ERF: r = std::erf(x); break;
      case LOG1P: r = std::log1p(x); break;
      case EXPM1: r = std::expm1(x); break;
      case SIGN: r = x != x ? x : static_cast<float>((x > 0.f) - (x < 0.f)); break;
      case FLOOR: r = std::floor(x); break;
      case CEIL: r = std::ceil(x); break;
      case SOFTPLUS: r = x > 20.f ? x : std::log1p(std::exp(x)); break;
      default: r = x;
    }
    d[i] = r;
  }
}

bool has_avx2() {
  static const bool ok = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
  return ok;
}

struct Program {
  const int32_t* code;
  int n_instr, n_in, n_out;
  const float* const* in;
  const int* in_scalar;
  const float* consts;
  float* const* out;
  const int* out_regs;
  long long n;
};

// runs blocks [b0, b1) of the program; `regs` is this thread's scratch of kMaxRegs blocks
void run_blocks(const Program& p, long long b0, long long b1, float* regs, float* cbuf) {
  const bool avx2 = has_avx2();
  for (long long blk = b0; blk < b1; ++blk) {
    const long long base = blk * kBlock;
    const int live = static_cast<int>(p.n - base < kBlock ? p.n - base : kBlock);
    // operand pointer of register r for this block
    auto operand = [&](int r, float* fill) -> const float* {
      if (r >= kConstBase) {
        const float v = p.consts[r - kConstBase];
        for (int i = 0; i < kBlock; ++i) fill[i] = v;
        return fill;
      }
      if (r < p.n_in) {
        if (p.in_scalar[r]) {
          const float v = p.in[r][0];
          for (int i = 0; i < kBlock; ++i) fill[i] = v;
          return fill;
        }
        if (live == kBlock) return p.in[r] + base;
        memcpy(fill, p.in[r] + base, sizeof(float) * live);       // the ragged last block is padded
        for (int i = live; i < kBlock; ++i) fill[i] = 1.f;
        return fill;
      }
      return regs + static_cast<size_t>(r) * kBlock;
    };
    for (int k = 0; k < p.n_instr; ++k) {
      const int32_t* ins = p.code + 4 * k;
      const int op = ins[0];
      float* d = regs + static_cast<size_t>(ins[1]) * kBlock;
      const float* a = operand(ins[2], cbuf);
      const float* b = op < NEG ? operand(ins[3], cbuf + kBlock) : a;
      if (avx2) run_instr_avx2(op, d, a, b);
      else run_instr_scalar(op, d, a, b);
    }
    for (int o = 0; o < p.n_out; ++o)
      memcpy(p.out[o] + base, regs + static_cast<size_t>(p.out_regs[o]) * kBlock, sizeof(float) * live);
  }
}

}  // namespace

// Runs an elementwise program over n values.  code: n_instr x {op, dst, a, b}; inputs: n_in float32 arrays
// (in_scalar[i] != 0: one value, broadcast); consts: the constants operands >= 2^20 name; outputs:
// n_out arrays receiving registers out_regs.  Returns 0, or -1 for a malformed program.
MIMIR_CPU_API int mimir_cpu_fused(const int32_t* code, int n_instr, const float* const* in, const int* in_scalar, int n_in,
                                  const float* consts, int n_consts, float* const* out, const int* out_regs, int n_out,
                                  long long n) {
  if (n_instr < 1 || n_instr > 256 || n_in < 0 || n_in > 16 || n_out < 1 || n < 0) return -1;
  for (int k = 0; k < n_instr; ++k) {
    const int32_t* ins = code + 4 * k;
    const bool binary = ins[0] >= ADD && ins[0] <= MIN, unary = ins[0] >= NEG && ins[0] <= SOFTPLUS;
    if (!binary && !unary) return -1;
    if (ins[1] < n_in || ins[1] >= kMaxRegs) return -1;
    for (int o = 2; o < (binary ? 4 : 3); ++o) {
      const int r = ins[o];
      if (r >= kConstBase) { if (r - kConstBase >= n_consts) return -1; }
      else if (r < 0 || r >= kMaxRegs) return -1;
    }
  }
  for (int o = 0; o < n_out; ++o)
    if (out_regs[o] < n_in || out_regs[o] >= kMaxRegs) return -1;
  if (n == 0) return 0;
  const Program p{code, n_instr, n_in, n_out, in, in_scalar, consts, out, out_regs, n};
  const long long blocks = (n + kBlock - 1) / kBlock;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  std::atomic<long long> next{0};
  const long long grain = blocks >= 64 * pool.size() ? 16 : 4;
  auto work = [&](int, int) {
    thread_local std::vector<float> scratch;
    if (scratch.size() < static_cast<size_t>(kMaxRegs + 2) * kBlock) scratch.resize(static_cast<size_t>(kMaxRegs + 2) * kBlock);
    float* regs = scratch.data();
    float* cbuf = regs + static_cast<size_t>(kMaxRegs) * kBlock;
    for (long long b0 = next.fetch_add(grain); b0 < blocks; b0 = next.fetch_add(grain))
      run_blocks(p, b0, b0 + grain < blocks ? b0 + grain : blocks, regs, cbuf);
  };
  if (blocks <= 8) work(0, 1);          // small tensors: not worth waking anyone
  else pool.run(work);
  return 0;
}
