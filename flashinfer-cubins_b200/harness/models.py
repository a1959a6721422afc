"""Model shapes the throughput cases draw from: published Hugging Face ``config.json``
constants, reduced to what the NVFP4 GEMM case lists need (the reference keeps a wider
table in ``harness/models.py:73-281``). Tokens are the GEMM's m; each linear layer
gives (n, k)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class Model:
    name: str
    hf: str
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    intermediate: int = 0  # dense MLP width; 0 when every layer is MoE
    experts: int = 0
    top_k: int = 0
    moe_intermediate: int = 0
    mla: dict[str, int] = field(default_factory=dict)  # multi-head latent attention ranks

    def get(self, key: str, default: Any = None) -> Any:
        return self.mla.get(key, default)

    def linear_shapes(self) -> dict[str, tuple[int, int]]:
        """GEMM (n, k) of every linear layer of one decoder layer."""
        out: dict[str, tuple[int, int]] = {}
        if self.mla:
            q_rank, kv_rank = self.mla["q_lora_rank"], self.mla["kv_lora_rank"]
            rope, nope, v = (self.mla[key] for key in
                             ("qk_rope_head_dim", "qk_nope_head_dim", "v_head_dim"))
            out["q_a_kv_a"] = (q_rank + kv_rank + rope, self.hidden)
            out["q_b"] = (self.heads * (nope + rope), q_rank)
            out["kv_b"] = (self.heads * (nope + v), kv_rank)
            out["o"] = (self.hidden, self.heads * v)
        else:
            out["qkv"] = ((self.heads + 2 * self.kv_heads) * self.head_dim, self.hidden)
            out["o"] = (self.hidden, self.heads * self.head_dim)
        if self.intermediate:
            out["gate_up"] = (2 * self.intermediate, self.hidden)
            out["down"] = (self.hidden, self.intermediate)
        if self.experts:
            out["expert_gate_up"] = (2 * self.moe_intermediate, self.hidden)
            out["expert_down"] = (self.hidden, self.moe_intermediate)
        return out


_TABLE = (
    #  name              hf repo                                   hidden heads kv  hd   inter  exp  topk moe_inter
    ("deepseek_v3", "deepseek-ai/DeepSeek-V3", 7168, 128, 128, 192, 18432, 256, 8, 2048),
    ("llama3_70b", "meta-llama/Llama-3.1-70B", 8192, 64, 8, 128, 28672, 0, 0, 0),
    ("llama3_405b", "meta-llama/Llama-3.1-405B", 16384, 128, 8, 128, 53248, 0, 0, 0),
    ("qwen3_32b", "Qwen/Qwen3-32B", 5120, 64, 8, 128, 25600, 0, 0, 0),
    ("qwen3_235b_a22b", "Qwen/Qwen3-235B-A22B", 4096, 64, 4, 128, 0, 128, 8, 1536),
    ("gpt_oss_120b", "openai/gpt-oss-120b", 2880, 64, 8, 64, 0, 128, 4, 2880),
    ("llama4_maverick", "meta-llama/Llama-4-Maverick-17B-128E", 5120, 40, 8, 128, 16384, 128, 1, 8192),
    ("mixtral_8x7b", "mistralai/Mixtral-8x7B-v0.1", 4096, 32, 8, 128, 0, 8, 2, 14336),
)
_MLA = {
    "deepseek_v3": dict(q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
                        qk_rope_head_dim=64, v_head_dim=128),
}

MODELS: dict[str, Model] = {
    row[0]: Model(*row, mla=_MLA.get(row[0], {})) for row in _TABLE
}
