// Option-string parser and validation shared by the Miir-style handle API and the tuning API.
#include "problem.h"

#include <cstdio>
#include <cstring>
#include <map>
#include <sstream>

namespace rb {
namespace {

// Tokeniser of the reference (ConvGenerator.cpp:82-98): a token containing "--" names a key (the text after it),
// the next token that does not is its value; later duplicates overwrite. Widened by one rule so that rocmlir-gen's
// single-dash flags (and therefore the text of a problem key) parse too: "-" followed by a letter is a key.
std::map<std::string, std::string> tokens(const char* arguments) {
  std::map<std::string, std::string> m;
  std::istringstream iss(arguments ? arguments : "");
  std::string tok, key;
  while (iss >> tok) {
    const size_t pos = tok.find("--");
    if (pos != std::string::npos) {
      key = tok.substr(pos + 2);
    } else if (tok.size() >= 2 && tok[0] == '-' && isalpha((unsigned char)tok[1])) {
      key = tok.substr(1);
    } else if (!key.empty()) {
      m[key] = tok;
      key.clear();
    }
  }
  return m;
}

bool to_long(const std::map<std::string, std::string>& m, const char* key, long long* out) {
  auto it = m.find(key);
  if (it == m.end()) return false;
  try {
    size_t used = 0;
    const long long v = std::stoll(it->second, &used);
    if (used != it->second.size()) return false;
    *out = v;
    return true;
  } catch (...) {
    return false;
  }
}

// absent: leaves *out alone and succeeds; present but malformed: fails
bool opt_int(const std::map<std::string, std::string>& m, const char* key, int* out) {
  if (!m.count(key)) return true;
  long long v;
  if (!to_long(m, key, &v) || v < -2147483647LL || v > 2147483647LL) return false;
  *out = (int)v;
  return true;
}

bool opt_bool(const std::map<std::string, std::string>& m, const char* key, int* out) {
  auto it = m.find(key);
  if (it == m.end()) return true;
  const std::string& v = it->second;
  if (v == "true" || v == "1") *out = 1;
  else if (v == "false" || v == "0") *out = 0;
  else return false;
  return true;
}

bool arch_is_ours(const std::string& arch) {
  return arch == "sm_100a" || arch == "sm_100" || arch == "nvptx64-nvidia-cuda:sm_100a" ||
         arch == "nvptx64-nvidia-cuda:sm_100";
}

// Miir's type names (ConvGenerator.cpp:569-589) and rocmlir-gen's (-t f16 ...)
int parse_type(const std::string& t) {
  if (t == "fp32" || t == "f32") return RB_F32;
  if (t == "fp16" || t == "f16") return RB_F16;
  if (t == "bf16") return RB_BF16;
  if (t == "i8") return RB_I8;
  if (t == "i32") return RB_I32;
  if (t == "fp8" || t == "f8E4M3FN" || t == "fp8_fp8") return RB_F8E4M3;
  if (t == "bf8" || t == "f8E5M2" || t == "bf8_bf8") return RB_F8E5M2;
  if (t == "fp8_bf8") return RB_F8E4M3_E5M2;
  if (t == "bf8_fp8") return RB_F8E5M2_E4M3;
  return -1;
}

// Layout translation of the reference (ConvGenerator.h:124-142) onto this library's letters.
// which: 0 filter (G N|K C H|Y|0 W|X|1 -> g k c y x), 1 input (n g c h w), 2 output (n g C|K h w -> n g k h w)
bool translate_layout(const std::string& src_in, int which, char out[8], bool unit_depth) {
  // Six letters name a third image dimension (D / Z / 2, ConvGenerator.cpp:622-627). With every depth equal to 1
  // that dimension has extent 1 and the tensor is the 2-D tensor on the same bytes, so the letter is dropped; a
  // real depth goes through rbConv3d, which this option grammar does not reach.
  std::string src = src_in;
  if (src.size() == 6 && unit_depth) {
    size_t hit = std::string::npos;
    for (size_t i = 0; i < 6; ++i) {
      const char ch = (char)tolower((unsigned char)src[i]);
      if (ch == 'd' || ch == 'z' || ch == '2') {
        if (hit != std::string::npos) return false;
        hit = i;
      }
    }
    if (hit == std::string::npos) return false;
    src.erase(hit, 1);
  }
  if (src.size() != 5) return false;
  for (size_t i = 0; i < 5; ++i) {
    const char ch = (char)tolower((unsigned char)src[i]);
    char o = 0;
    if (which == 0) {
      switch (ch) {
        case 'g': o = 'g'; break;
        case 'n': case 'k': o = 'k'; break;
        case 'c': o = 'c'; break;
        case 'h': case 'y': case '0': o = 'y'; break;
        case 'w': case 'x': case '1': o = 'x'; break;
      }
    } else {
      switch (ch) {
        case 'n': o = 'n'; break;
        case 'g': o = 'g'; break;
        case 'c': o = which == 1 ? 'c' : 'k'; break;
        case 'k': o = which == 2 ? 'k' : 0; break;
        case 'h': case '0': o = 'h'; break;
        case 'w': case '1': o = 'w'; break;
      }
    }
    if (!o) return false;
    for (size_t j = 0; j < i; ++j)
      if (out[j] == o) return false;
    out[i] = o;
  }
  out[5] = 0;
  return true;
}

long long out_dim(long long in, long long fil, long long pl, long long pr, long long stride, long long dil) {
  // ConvGenerator.h:98-104
  return (in + pl + pr - (fil - 1) * dil - 1) / stride + 1;
}

bool parse_conv(const std::map<std::string, std::string>& m, int direction, ProblemDesc* h) {
  static const char* required[] = {"batchsize", "groupsize", "in_layout", "in_type", "in_channels", "in_h", "in_w",
                                   "out_layout", "out_type", "out_channels", "out_h", "out_w", "fil_layout",
                                   "fil_type", "fil_w", "fil_h"};
  for (const char* k : required)
    if (!m.count(k)) return false;
  RbConvProblem& c = h->conv;
  memset(&c, 0, sizeof(c));
  const int in_t = parse_type(m.at("in_type")), fil_t = parse_type(m.at("fil_type")), out_t = parse_type(m.at("out_type"));
  const bool f8 = in_t == RB_F8E4M3 || in_t == RB_F8E5M2;
  if (in_t < 0 || fil_t < 0 || out_t < 0 || in_t == RB_I32 || in_t != fil_t || in_t > RB_F8E5M2) return false;
  if (in_t == RB_I8) {
    if (out_t != RB_I32) return false;   // i8 x i8 accumulates and stores i32
  } else if (f8) {
    if (out_t != RB_F32) return false;   // 8-bit floats accumulate and store f32
  } else if (out_t != in_t) {
    return false;
  }
  // ConvGenerator.cpp:631-638: 8-bit types run forward only
  if (direction != 0 && (in_t == RB_I8 || f8)) return false;
  c.data_type = in_t;
  c.direction = direction;
  // depth keys are optional (ConvGenerator.cpp:642-650); anything but 1 has no kernel behind this grammar
  bool unit_depth = true;
  for (const char* key : {"in_d", "fil_d", "out_d", "conv_stride_d", "dilation_d"}) {
    int v = 1;
    if (!opt_int(m, key, &v) || v <= 0) return false;
    if (v != 1 && (std::string(key) == "in_d" || std::string(key) == "fil_d" || std::string(key) == "out_d")) unit_depth = false;
  }
  int pad_d = 0;
  if (!opt_int(m, "padding_d", &pad_d) || pad_d < 0) return false;
  if (pad_d != 0) unit_depth = false;
  if (!unit_depth) return false;
  if (m.at("fil_layout").size() != m.at("in_layout").size() || m.at("in_layout").size() != m.at("out_layout").size())
    return false;   // the three tensors have the same number of image dimensions
  if (!translate_layout(m.at("fil_layout"), 0, c.fil_layout, unit_depth) ||
      !translate_layout(m.at("in_layout"), 1, c.in_layout, unit_depth) ||
      !translate_layout(m.at("out_layout"), 2, c.out_layout, unit_depth))
    return false;
  long long n, g, ci, co, ih, iw, oh, ow, fh, fw;
  if (!to_long(m, "batchsize", &n) || !to_long(m, "groupsize", &g) || !to_long(m, "in_channels", &ci) ||
      !to_long(m, "out_channels", &co) || !to_long(m, "in_h", &ih) || !to_long(m, "in_w", &iw) ||
      !to_long(m, "out_h", &oh) || !to_long(m, "out_w", &ow) || !to_long(m, "fil_h", &fh) || !to_long(m, "fil_w", &fw))
    return false;
  if (n <= 0 || g <= 0 || ci <= 0 || co <= 0 || ih <= 0 || iw <= 0 || oh <= 0 || ow <= 0 || fh <= 0 || fw <= 0) return false;
  if (ci % g || co % g) return false;
  const long long lim = 0x7fffffffLL;
  if (n > lim || ci > lim || co > lim || ih > lim || iw > lim || fh > lim || fw > lim) return false;
  c.n = (int)n; c.g = (int)g; c.c = (int)(ci / g); c.k = (int)(co / g);
  c.h = (int)ih; c.w = (int)iw; c.y = (int)fh; c.x = (int)fw;
  c.stride_h = c.stride_w = c.dil_h = c.dil_w = 1;
  int pad_h = 0, pad_w = 0;
  if (!opt_int(m, "dilation_h", &c.dil_h) || !opt_int(m, "dilation_w", &c.dil_w) ||
      !opt_int(m, "conv_stride_h", &c.stride_h) || !opt_int(m, "conv_stride_w", &c.stride_w) ||
      !opt_int(m, "padding_h", &pad_h) || !opt_int(m, "padding_w", &pad_w))
    return false;
  if (c.dil_h <= 0 || c.dil_w <= 0 || c.stride_h <= 0 || c.stride_w <= 0 || pad_h < 0 || pad_w < 0) return false;
  c.pad_h = c.pad_h_r = pad_h;   // one key sets both sides (ConvGenerator.cpp:598-601)
  c.pad_w = c.pad_w_r = pad_w;
  // dimension checks of ConvGenerator.cpp:221-245
  if (out_dim(ih, fh, pad_h, pad_h, c.stride_h, c.dil_h) != oh || out_dim(iw, fw, pad_w, pad_w, c.stride_w, c.dil_w) != ow)
    return false;
  if (ih + 2 * pad_h < fh || iw + 2 * pad_w < fw) return false;
  c.ho = (int)oh;
  c.wo = (int)ow;
  h->kind = kConv;
  return true;
}

bool parse_gemm(const std::map<std::string, std::string>& m, ProblemDesc* h) {
  RbGemmProblem& p = h->gemm;
  memset(&p, 0, sizeof(p));
  if (!m.count("t") || !m.count("m") || !m.count("n") || !m.count("k")) return false;
  const int t = parse_type(m.at("t"));
  if (t < 0 || t == RB_I32) return false;
  // rocmlir-gen.cpp:430-455: -t i8 defaults to an i32 result, 8-bit floats to an f32 result
  int out_t = (t == RB_I8) ? RB_I32 : (t >= RB_F8E4M3 ? RB_F32 : t);
  if (m.count("out_datatype")) out_t = parse_type(m.at("out_datatype"));
  if (out_t < 0 || out_t > RB_F8E4M3) return false;
  p.g = 1;
  if (!opt_int(m, "g", &p.g) || !opt_int(m, "m", &p.m) || !opt_int(m, "n", &p.n) || !opt_int(m, "k", &p.k)) return false;
  if (!opt_bool(m, "transA", &p.trans_a) || !opt_bool(m, "transB", &p.trans_b) || !opt_bool(m, "transC", &p.trans_c))
    return false;
  if (p.g <= 0 || p.m <= 0 || p.n <= 0 || p.k <= 0) return false;
  p.ab_type = t;
  p.c_type = out_t;
  h->kind = kGemm;
  return true;
}

bool parse_attention(const std::map<std::string, std::string>& m, ProblemDesc* h) {
  RbAttentionProblem& p = h->att;
  memset(&p, 0, sizeof(p));
  if (!m.count("t") || !m.count("seq_len_q") || !m.count("seq_len_k") || !m.count("head_dim_qk") || !m.count("head_dim_v"))
    return false;
  const int t = parse_type(m.at("t"));
  if (!(t == RB_F16 || t == RB_BF16)) return false;
  p.g = 1;
  if (!opt_int(m, "g", &p.g) || !opt_int(m, "seq_len_q", &p.seq_q) || !opt_int(m, "seq_len_k", &p.seq_k) ||
      !opt_int(m, "head_dim_qk", &p.head_qk) || !opt_int(m, "head_dim_v", &p.head_v))
    return false;
  if (!opt_bool(m, "transQ", &p.trans_q) || !opt_bool(m, "transK", &p.trans_k) || !opt_bool(m, "transV", &p.trans_v) ||
      !opt_bool(m, "transO", &p.trans_o) || !opt_bool(m, "causal", &p.causal))
    return false;
  if (m.count("with-attn-scale")) {
    // rocmlir-gen's flag is a boolean that adds a [G,Sq,Sk] scale tensor; here it carries the scalar itself
    try {
      p.scale = std::stof(m.at("with-attn-scale"));
      p.has_scale = 1;
    } catch (...) {
      return false;
    }
  }
  if (p.g <= 0 || p.seq_q <= 0 || p.seq_k <= 0) return false;
  if (p.head_qk % 8 || p.head_qk > 128 || p.head_qk <= 0 || p.head_v % 8 || p.head_v > 128 || p.head_v <= 0) return false;
  p.data_type = t;
  h->kind = kAttention;
  return true;
}

}  // namespace

// Strings of the reference's accelerated GEMM / convolution parameters (Serializable.h:64-131, RockAttrDefs.td:300-434):
//   v2:MPerBlock,NPerBlock,KpackPerBlock,MPerWave,NPerWaveOrMnPerXdl,KPack,SplitKFactor,ForceUnroll,ThreadCopyMore
// and the un-prefixed version 1 with the same fields minus SplitKFactor. They describe an MFMA tiling; what carries
// over to this hardware is the block tile and the K split: MPerBlock picks one CTA (<= 128 rows) or a CTA pair,
// NPerBlock the nearest tile width not below it (64 / 128 / 256), SplitKFactor is honoured as given; the wave-level
// fields have no counterpart and are only checked for sanity. Anything else fails applicability.
static bool reference_perf_config_to_variant(const char* str, uint32_t* variant) {
  const bool v2 = strncmp(str, "v2:", 3) == 0;
  const char* body = v2 ? str + 3 : str;
  int f[9] = {0, 0, 0, 0, 0, 0, 1, 0, 0}, n = 0;
  const char* q = body;
  while (n < 9) {
    char* end = nullptr;
    const long v = strtol(q, &end, 10);
    if (end == q || v < 0 || v > (1 << 20)) return false;
    f[n++] = (int)v;
    if (*end == '\0') break;
    if (*end != ',') return false;
    q = end + 1;
    if (n == 9) return false;   // a tenth field
  }
  if (v2 ? (n < 7 || n > 9) : n != 8) return false;   // Serializable.h:72-80: six to eight commas for v2
  if (!v2) { f[8] = f[7]; f[7] = f[6]; f[6] = 1; }     // version 1 has no SplitKFactor
  const int m_per_block = f[0], n_per_block = f[1], kpack_per_block = f[2], kpack = f[5], split_k = f[6];
  if (m_per_block <= 0 || n_per_block <= 0 || kpack_per_block <= 0 || kpack <= 0 || split_k <= 0 || split_k > 255) return false;
  if (m_per_block > 256 || n_per_block > 256) return false;
  const uint32_t ctas = m_per_block <= 128 ? 1u : 2u;
  const uint32_t bn_code = n_per_block <= 64 ? 1u : n_per_block <= 128 ? 2u : 3u;
  *variant = ctas | (bn_code << 12) | ((uint32_t)split_k << 16);
  return true;
}

bool perf_config_to_variant(const char* str, uint32_t* variant) {
  if (!str || !variant) return false;
  if (strncmp(str, "b200:", 5) != 0) return reference_perf_config_to_variant(str, variant);
  int tm = 0, tn = 0, stages = 0, splits = 0, sk = 0, kpr = 0;
  char tail = 0;
  const int got = sscanf(str, "b200:%d,%d,%d,%d,%d,%d%c", &tm, &tn, &stages, &splits, &sk, &kpr, &tail);
  if (got != 5 && got != 6) return false;
  if (got == 5) {   // a sixth field must not be half there ("...,0," or trailing junk)
    int commas = 0;
    for (const char* c = str; *c; ++c) commas += *c == ',';
    const char last = str[strlen(str) - 1];
    if (commas != 4 || last < '0' || last > '9') return false;
  }
  if (!(tm == 128 || tm == 256) || !(tn == 64 || tn == 128 || tn == 256)) return false;
  if (stages < 0 || stages > 15 || splits < 0 || splits > 255 || !(sk == 0 || sk == 1)) return false;
  if (!(kpr == 0 || kpr == 1 || kpr == 2 || kpr == 4)) return false;
  const uint32_t bn_code = tn == 64 ? 1u : tn == 128 ? 2u : 3u;
  const uint32_t kpr_code = kpr == 0 ? 0u : kpr == 1 ? 1u : kpr == 2 ? 2u : 3u;
  *variant = (tm == 256 ? 2u : 1u) | ((uint32_t)stages << 4) | ((uint32_t)sk << 9) | (bn_code << 12) |
             ((uint32_t)splits << 16) | (kpr_code << 28);
  return true;
}

std::string variant_to_perf_config(uint32_t v) {
  const int ctas = (v & 0xF) == 1 ? 1 : 2;
  const int bn_code = (v >> 12) & 0xF;
  const int tn = bn_code == 1 ? 64 : bn_code == 2 ? 128 : 256;
  const int kpr_code = (v >> 28) & 3;
  char buf[64];
  int len = snprintf(buf, sizeof(buf), "b200:%d,%d,%d,%d,%d", ctas == 2 ? 256 : 128, tn, (int)((v >> 4) & 0xF),
                     (int)((v >> 16) & 0xFF), (int)((v >> 9) & 1));
  if (kpr_code) snprintf(buf + len, sizeof(buf) - len, ",%d", kpr_code == 1 ? 1 : kpr_code == 2 ? 2 : 4);
  return buf;
}

bool refresh_problem(ProblemDesc* d) {
  bool ok = true;
  // applicability: the library must have a plan for the problem (layouts, sizes, types) under this variant
  const int saved_variant = rbGetGemmVariant();
    rbSetGemmVariant((int)d->variant);
  if (d->kind == kConv) {
    RbGemmProblem gp;
    ok = rbConvGetGemmProblem(&d->conv, &gp) == RB_SUCCESS;
    if (ok) d->workspace = rbConvWorkspaceSize(&d->conv);
  } else if (d->kind == kGemm) {
    RbGemmConfigInfo info;
    ok = rbGemmGetConfig(&d->gemm, &info) == RB_SUCCESS;
    if (ok) d->workspace = rbGemmWorkspaceSize(&d->gemm);
  } else {
    d->workspace = 0;
  }
  rbSetGemmVariant(saved_variant);
  return ok;
}

bool parse_problem(const char* options, ProblemDesc* h) {
  if (!options || !h) return false;
  const auto m = tokens(options);
  auto arch = m.find("arch");
  if (arch == m.end() || !arch_is_ours(arch->second)) return false;
  auto op = m.find("operation");
  if (op == m.end()) return false;
  h->arch = arch->second;
  bool ok = false;
  if (op->second == "conv") ok = parse_conv(m, 0, h);
  else if (op->second == "conv_bwd_data") ok = parse_conv(m, 1, h);
  else if (op->second == "conv_bwd_weight") ok = parse_conv(m, 2, h);
  else if (op->second == "gemm") ok = parse_gemm(m, h);
  else if (op->second == "attention") ok = parse_attention(m, h);
  if (!ok) return false;
  if (!opt_int(m, "kernel_id", &h->kernel_id) || !opt_int(m, "num_cu", &h->num_cu)) return false;
  if (m.count("kernel_name")) h->kernel_name = m.at("kernel_name");
  h->variant = 0;
  if (m.count("perf_config")) {
    h->perf_config = m.at("perf_config");
    if (!perf_config_to_variant(h->perf_config.c_str(), &h->variant)) return false;
  }
  return refresh_problem(h);
}

}  // namespace rb
