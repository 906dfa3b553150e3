"""The model shapes of the verify window (no device code, no torch): shared by the runner and by host-only tools."""
from dataclasses import dataclass, field


@dataclass
class StackShape:
    """The whole model's shapes (the benchmark configurations' defaults)."""
    n: int = 3072
    nexp: int = 512
    topk: int = 10
    ff: int = 768
    nkh: int = 16
    nvh: int = 48
    nq: int = 24
    nkv: int = 4
    hd: int = 256
    nrot: int = 64
    vocab: int = 151936
    kinds: list = field(default_factory=lambda: [0, 0, 0, 1, 0, 0, 0, 1])   # 0 DeltaNet, 1 attention
    ctx: int = 32768
    kv_slack: int = 64   # positions the K/V cache holds past ctx (the tokens a run appends)
    eps: float = 1e-6
    rope_base: float = 1e7
    sigma: float = 0.02
    experts: str = "q4k"   # routed experts: "q4k" (Q4_K gate|up, Q6_K down) or "q8_0" (both Q8_0)
    hc: int = 1            # residual streams: 1 = plain residual + RMS norm; > 1 = hyper-connections (reads mix the streams)
    hc_lr: int = 320       # the hyper-connections' low rank
    draft: bool = False    # the stack is a draft (MTP) layer: its streams come from a window's rows and the next tokens' embeddings
    qsa_top: int = 0       # blocks of 4 positions an attention row keeps (the reference: 512); 0: no block selection, every position attended
    kv_q8: bool = False    # K/V rows as int8 in groups of 32 with f16 scales (the reference's kv_q8) instead of f16
