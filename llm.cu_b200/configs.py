"""Named model shapes: the reference's literals (LLaMA3-8B) and the other benchmark shapes."""
from dataclasses import dataclass


@dataclass(frozen=True)
class ModelConfig:
    name: str
    n_layers: int
    d_model: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    rope_theta: float = 500000.0
    eps: float = 1e-5
    bf16_weights: bool = True  # drawn as BF16 and converted to FP16 at load, as the reference does
    embed_rows: int = 0        # rows of the embedding table actually materialised (0 = vocab)

    @property
    def q_rows(self):
        return self.n_q_heads * self.head_dim

    @property
    def kv_rows(self):
        return self.n_kv_heads * self.head_dim

    def matmul_params(self):
        per_layer = (self.q_rows + 2 * self.kv_rows) * self.d_model + self.d_model * self.q_rows \
            + 3 * self.ffn * self.d_model
        return per_layer * self.n_layers

    def weight_bytes_per_token(self, tp=1):
        """Bytes of weights one decoded token must stream on each of `tp` tensor-parallel GPUs:
        its share of the projections and of lm_head, plus the replicated norm gains and one
        embedding row."""
        norms = (2 * self.n_layers + 1) * self.d_model
        return 2 * ((self.matmul_params() + self.vocab * self.d_model) // tp + norms) + 2 * self.d_model

    def kv_bytes_per_position(self):
        return 2 * 2 * self.kv_rows * self.n_layers

    def decode_bytes(self, cached_positions, tp=1):
        """Algorithmic bytes, per GPU, of one decode step that attends over `cached_positions` rows and
        appends one (the KV cache is split by KV head across `tp` GPUs)."""
        return self.weight_bytes_per_token(tp) + self.kv_bytes_per_position() // tp * (cached_positions + 1)


CONFIGS = {
    # 2-layer plumbing model; FP16 weights drawn directly
    "tiny": ModelConfig("tiny", 2, 256, 4, 2, 64, 768, 4096, bf16_weights=False),
    # the reference's hard-coded shape
    "llama3_8b": ModelConfig("llama3_8b", 32, 4096, 32, 8, 128, 14336, 128256),
    # 8B layer shape, two layers, small embedding table: small enough to run through the reference
    # binary and the CPU oracle in seconds; used to pin the oracle against the reference itself
    "llama3_8b_l2": ModelConfig("llama3_8b_l2", 2, 4096, 32, 8, 128, 14336, 128256, embed_rows=1024),
    # 8B layer shape cut down to ~2.3 GB (4 layers, 32K vocabulary) for multi-pass profiler captures
    "llama3_8b_prof": ModelConfig("llama3_8b_prof", 4, 4096, 32, 8, 128, 14336, 32768),
    "llama3_70b": ModelConfig("llama3_70b", 80, 8192, 64, 8, 128, 28672, 128256),
    # 70B layer shape, two layers, small embedding table: the parity case of the 70B shape (the CPU oracle runs
    # it in seconds; under tensor parallelism each of 8 GPUs holds one KV head and 8 query heads)
    "llama3_70b_l2": ModelConfig("llama3_70b_l2", 2, 8192, 64, 8, 128, 28672, 128256, embed_rows=1024),
}
