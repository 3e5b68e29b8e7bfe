// CPU GRPO objective (oracle and CPU path): same definition as csrc/sm100/grpo_loss.cu,
// written serially with libm exp.
#include <algorithm>
#include <cmath>

extern "C" {

int ka_cpu_grpo_advantages(const float* rewards, float* adv, int n_groups, int group, float eps) {
  for (int g = 0; g < n_groups; ++g) {
    const float* r = rewards + static_cast<long long>(g) * group;
    float sum = 0.f;
    for (int i = 0; i < group; ++i) sum += r[i];
    const float mean = sum / static_cast<float>(group);
    float ss = 0.f;
    for (int i = 0; i < group; ++i) ss = std::fmaf(r[i] - mean, r[i] - mean, ss);
    const float var = group > 1 ? ss / static_cast<float>(group - 1) : 0.f;
    const float inv = 1.0f / (std::sqrt(var) + eps);
    for (int i = 0; i < group; ++i) adv[static_cast<long long>(g) * group + i] = (r[i] - mean) * inv;
  }
  return 0;
}

// grad: d loss / d logp_new per token (already normalised); out: loss, clip fraction, tokens.
int ka_cpu_grpo_loss(const float* logp_new, const float* logp_old, const float* logp_ref, const float* adv,
                     const unsigned char* mask, int n_seq, int seq_len, float eps_low, float eps_high, float beta,
                     int seq_mean, float* grad, float* out) {
  double total = 0, count = 0, clip = 0, mean_acc = 0, valid_seq = 0;
  for (int s = 0; s < n_seq; ++s) {
    double ssum = 0, scnt = 0;
    for (int t = 0; t < seq_len; ++t) {
      const long long i = static_cast<long long>(s) * seq_len + t;
      grad[i] = 0.f;
      if (mask && !mask[i]) continue;
      const float ratio = std::exp(logp_new[i] - logp_old[i]);
      const float s1 = ratio * adv[s];
      const float s2 = std::min(std::max(ratio, 1.f - eps_low), 1.f + eps_high) * adv[s];
      const bool unclipped = s1 <= s2;
      float loss = -(unclipped ? s1 : s2);
      float g = unclipped ? -s1 : 0.f;
      if (beta > 0.f && logp_ref) {
        const float d = logp_ref[i] - logp_new[i];
        const float e = std::exp(d);
        loss += beta * (e - d - 1.f);
        g += beta * (1.f - e);
      }
      grad[i] = g;
      ssum += loss;
      scnt += 1;
      clip += unclipped ? 0 : 1;
    }
    total += ssum;
    count += scnt;
    if (scnt > 0) {
      mean_acc += ssum / scnt;
      valid_seq += 1;
    }
    // stash the count in out-of-band fashion: second pass below
  }
  for (int s = 0; s < n_seq; ++s) {
    double scnt = 0;
    for (int t = 0; t < seq_len; ++t) {
      const long long i = static_cast<long long>(s) * seq_len + t;
      if (!mask || mask[i]) scnt += 1;
    }
    const double w = seq_mean ? (scnt > 0 ? 1.0 / (scnt * valid_seq) : 0.0) : (count > 0 ? 1.0 / count : 0.0);
    for (int t = 0; t < seq_len; ++t) grad[static_cast<long long>(s) * seq_len + t] *= static_cast<float>(w);
  }
  out[0] = static_cast<float>(seq_mean ? (valid_seq > 0 ? mean_acc / valid_seq : 0.0) : (count > 0 ? total / count : 0.0));
  out[1] = static_cast<float>(count > 0 ? clip / count : 0.0);
  out[2] = static_cast<float>(count);
  return 0;
}

}  // extern "C"
