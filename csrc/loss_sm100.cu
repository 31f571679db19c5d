// Token-level policy-loss kernels: the PPO clipped surrogate (with optional dual clip) and its gradient in one
// pass, instead of a chain of elementwise PyTorch kernels per micro-batch.  Per token, with kl = old_logp - logp
// (or the sequence-level quantity GSPO substitutes for it) and r = exp(-kl):
//   loss = max(-r A, -clip(r, 1 - e_lo, 1 + e_hi) A)            (dual clip: for A < 0, min(that, -c A))
//   clip = 1 if the clipped branch is the larger one
//   dkl  = d loss / d kl  (r A on the unclipped branch, 0 on the clipped / dual-clipped ones)
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_utils.h"

namespace rb {

__global__ void policy_loss_fwd_kernel(const float* __restrict__ ppo_kl, const float* __restrict__ adv,
                                       float* __restrict__ loss, float* __restrict__ clipfrac, float* __restrict__ dkl,
                                       long long n, float e_lo, float e_hi, float c_dual) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float kl = ppo_kl[i];
    const float r = __expf(-kl);
    const float a = adv[i];
    const float l1 = -r * a;
    const float rc = fminf(fmaxf(r, 1.f - e_lo), 1.f + e_hi);
    const float l2 = -rc * a;
    float l = fmaxf(l1, l2);
    // d(-r a)/dkl = r a on the unclipped branch; the clipped value does not depend on kl unless the clamp is
    // inactive (then l1 == l2 and the same gradient applies)
    float g = (l1 >= l2 || rc == r) ? r * a : 0.f;
    if (c_dual > 1.f && a < 0.f) {
      const float l3 = -c_dual * a;
      if (l3 < l) { l = l3; g = 0.f; }
    }
    loss[i] = l;
    clipfrac[i] = (l2 > l1) ? 1.f : 0.f;
    dkl[i] = g;
  }
}

}  // namespace rb

extern "C" int rb_policy_loss(const float* ppo_kl, const float* adv, float* loss, float* clipfrac, float* dkl, long long n,
                              float eps_clip, float eps_clip_high, float eps_clip_c, cudaStream_t st) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > rb::num_sms() * 8LL) blocks = rb::num_sms() * 8LL;
  rb::policy_loss_fwd_kernel<<<(int)blocks, 256, 0, st>>>(ppo_kl, adv, loss, clipfrac, dkl, n, eps_clip, eps_clip_high,
                                                         eps_clip_c);
  rb_note_launch(1);
  return (int)cudaGetLastError();
}
