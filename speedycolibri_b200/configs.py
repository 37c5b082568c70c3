"""The five benchmark shapes (and small test shapes) of the routed-expert MoE block."""
from __future__ import annotations

from dataclasses import dataclass, replace

FMT_E4M3_ROW = 4
FMT_NVFP4 = 5
FMT_MXFP4 = 6
FMT_FP8_B128 = 8
SCORE_SOFTMAX = 0
SCORE_SIGMOID = 1


@dataclass(frozen=True)
class MoeShape:
    name: str
    H: int                 # hidden
    E: int                 # routed experts
    k: int                 # top-k
    I: int                 # expert (and shared-expert) intermediate
    T: int                 # tokens per block call
    fmt: int = FMT_NVFP4
    score: int = SCORE_SOFTMAX
    norm_topk: bool = False
    routed_scale: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    shared: bool = True
    select_bias_std: float = 0.0   # sigmoid selection bias ~ N(0, std)
    zipf_s: float = 0.0            # > 0: additive logit bias giving Zipf(s) expert popularity
    block_spread: float = 0.0      # > 0: every 128x128 weight block is scaled by exp(N(0, spread)) (host generation)
    note: str = ""

    def with_tokens(self, T: int) -> "MoeShape":
        return replace(self, T=T)

    # ---- algorithmic work of one block call (what the roofline figures use) ----
    def matrix_bytes(self, O: int, K: int) -> int:
        """Packed bytes of one [O,K] weight matrix (crates/colibri-core/src/quant.rs:762-766)."""
        if self.fmt == FMT_NVFP4:
            return O * ((K + 1) // 2) + O * ((K + 15) // 16) + 4
        if self.fmt == FMT_MXFP4:
            return O * ((K + 1) // 2) + O * ((K + 31) // 32) + 4
        if self.fmt == FMT_FP8_B128:
            return O * K + 4 * ((O + 127) // 128) * ((K + 127) // 128)
        return O * K + 4 * O

    def expert_bytes(self) -> int:
        return 2 * self.matrix_bytes(self.I, self.H) + self.matrix_bytes(self.H, self.I)

    def flops(self, T: int | None = None) -> int:
        T = self.T if T is None else T
        return 2 * T * self.E * self.H + 6 * self.H * self.I * (T * self.k + (T if self.shared else 0))

    def bytes_moved(self, active_experts: int, T: int | None = None) -> int:
        """Weights of the distinct active experts (routed + shared) + router + x in + out."""
        T = self.T if T is None else T
        n = active_experts + (1 if self.shared else 0)
        return n * self.expert_bytes() + 2 * self.E * self.H + 4 * T * self.H


CONFIGS = {
    "c0": MoeShape("c0", H=1024, E=32, k=4, I=512, T=128, norm_topk=True,
                   note="CPU-runnable single layer, softmax top-4 renormalised, NVFP4"),
    "c1": MoeShape("c1", H=2048, E=128, k=8, I=768, T=8,
                   note="decode shape (T in 1,4,8), softmax top-8, NVFP4"),
    "c2": MoeShape("c2", H=2048, E=128, k=8, I=768, T=512, fmt=FMT_FP8_B128,
                   note="prefill shape, FP8 E4M3 with f32 scale per 128x128 block"),
    "c3": MoeShape("c3", H=7168, E=256, k=8, I=2048, T=4096, score=SCORE_SIGMOID, norm_topk=True,
                   routed_scale=2.5, n_group=8, topk_group=4, select_bias_std=0.01,
                   note="large expert-parallel layer, sigmoid group-limited routing, NVFP4"),
    "c4": MoeShape("c4", H=6144, E=384, k=8, I=2048, T=16384, shared=False, zipf_s=1.2,
                   note="skewed load, softmax top-8 + Zipf(1.2) logit bias, NVFP4, no shared expert"),
    # c3 with 32 experts and 512 tokens: same matrices and rows/expert, 0.8 GB of weights — the
    # small case that ncu captures are taken on
    "c3s": MoeShape("c3s", H=7168, E=32, k=8, I=2048, T=512, score=SCORE_SIGMOID, norm_topk=True,
                    routed_scale=2.5, n_group=8, topk_group=4, select_bias_std=0.01,
                    note="c3 shapes at 1/8 of the experts and tokens (profiling case)"),
    # c4 with 48 experts and 2048 tokens: same matrices, skew and rows/expert (1 GB of weights)
    "c4s": MoeShape("c4s", H=6144, E=48, k=8, I=2048, T=2048, shared=False, zipf_s=1.2,
                    note="c4 shapes at 1/8 of the experts and tokens (profiling case)"),
    # c3's router (H, E, routing rule, T) over experts of 1/16 of the width: the profiling case of the router kernels
    "c3r": MoeShape("c3r", H=7168, E=256, k=8, I=128, T=4096, score=SCORE_SIGMOID, norm_topk=True,
                    routed_scale=2.5, n_group=8, topk_group=4, select_bias_std=0.01,
                    note="c3's router with thin experts (profiling case)"),
    # small shapes for tests
    "tiny": MoeShape("tiny", H=64, E=8, k=2, I=32, T=5, norm_topk=True),
    "tiny_sig": MoeShape("tiny_sig", H=128, E=16, k=4, I=64, T=37, score=SCORE_SIGMOID, norm_topk=True,
                         routed_scale=2.5, n_group=4, topk_group=2, select_bias_std=0.05),
    "tiny_fp8": MoeShape("tiny_fp8", H=256, E=8, k=2, I=128, T=19, fmt=FMT_FP8_B128),
    # prefill-sized segments (tcgen05 path), small enough for host generation
    "mid": MoeShape("mid", H=512, E=8, k=2, I=256, T=512, norm_topk=True),
    "mid_ragged": MoeShape("mid_ragged", H=320, E=6, k=2, I=192, T=333, shared=False),
    # FP8 on the tcgen05 path: block scales that differ by orders of magnitude inside a row block,
    # ragged K / feature counts, and the per-row scaled form
    "mid_fp8": MoeShape("mid_fp8", H=512, E=8, k=2, I=256, T=512, fmt=FMT_FP8_B128, block_spread=1.5),
    "mid_fp8_ragged": MoeShape("mid_fp8_ragged", H=320, E=6, k=2, I=192, T=333, shared=False, fmt=FMT_FP8_B128,
                               block_spread=1.5),
    "mid_fp8row": MoeShape("mid_fp8row", H=256, E=4, k=2, I=128, T=100, fmt=FMT_E4M3_ROW, block_spread=1.0),
    # MXFP4 (E8M0 scale per 32): register-level and tcgen05 kernel families
    "tiny_mx": MoeShape("tiny_mx", H=128, E=8, k=2, I=64, T=21, fmt=FMT_MXFP4, norm_topk=True),
    "mid_mx": MoeShape("mid_mx", H=512, E=8, k=2, I=256, T=512, fmt=FMT_MXFP4, norm_topk=True, block_spread=1.0),
    "tiny_zipf": MoeShape("tiny_zipf", H=64, E=16, k=4, I=32, T=70, shared=False, zipf_s=1.2),
}
