"""Model shapes of the benchmark configurations (qwen35 hybrid, one MTP layer)."""
from .binding import ModelConfig

MODEL_SEED = 0x5EED
PROMPT_SEED = 0xC0FFEE


def tiny():
    """4 layers (DeltaNet x3, attention), hidden 256, 4q/2kv x 64, DeltaNet 2k/4v x 64, FFN 512, vocab 4096."""
    return ModelConfig(n_layers=4, n_embd=256, n_ff=512, n_heads=4, n_kv_heads=2, head_dim=64, rope_dim=16,
                       rope_theta=1e7, rms_eps=1e-6, ssm_conv_kernel=4, ssm_num_k_heads=2, ssm_num_v_heads=4,
                       ssm_head_dim=64, full_attention_interval=4, vocab_size=4096, mtp_layers=1, weight_sigma=0.02)


def qwen27b(n_layers=64):
    """27B-class shape: 64 layers (every 4th full attention), hidden 5120, 24q/4kv x 256,
    DeltaNet 16k/48v x 128 conv 4, FFN 17408, vocab 151936."""
    return ModelConfig(n_layers=n_layers, n_embd=5120, n_ff=17408, n_heads=24, n_kv_heads=4, head_dim=256, rope_dim=64,
                       rope_theta=1e7, rms_eps=1e-6, ssm_conv_kernel=4, ssm_num_k_heads=16, ssm_num_v_heads=48,
                       ssm_head_dim=128, full_attention_interval=4, vocab_size=151936, mtp_layers=1, weight_sigma=0.02)
