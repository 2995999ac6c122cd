"""Random-init Llama of TinyLlama-1.1B's attention shape (hidden 2048, 32 query heads over 4 KV heads of 64,
vocabulary 32000) used by the end-to-end wrapper fixture and its parity test.  The weights come from an
explicit CPU generator, parameter by parameter in name order, so that the reference run that produced the
fixture and the test see the same model."""
import numpy as np
import torch


def tiny_llama(num_layers: int, seed: int = 1234, vocab: int = 32000):
    import transformers
    cfg = transformers.LlamaConfig(vocab_size=vocab, hidden_size=2048, intermediate_size=5632,
                                   num_hidden_layers=num_layers, num_attention_heads=32, num_key_value_heads=4,
                                   max_position_embeddings=2048, rms_norm_eps=1e-5, rope_theta=10000.0,
                                   tie_word_embeddings=False, bos_token_id=1, eos_token_id=2, pad_token_id=None)
    cfg._attn_implementation = "eager"
    model = transformers.LlamaForCausalLM(cfg).float().eval()
    g = torch.Generator(device="cpu").manual_seed(seed)
    with torch.no_grad():
        for name, p in sorted(model.named_parameters(), key=lambda kv: kv[0]):
            if p.dim() >= 2:
                p.copy_(torch.empty(p.shape, dtype=torch.float32).normal_(0.0, 0.02, generator=g))
            else:
                p.fill_(1.0)
    return model


def prompts(batch: int, length: int, seed: int = 7, vocab: int = 32000) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(3, vocab, (batch, length), generator=g)


def probe_columns(count: int = 256, seed: int = 11, vocab: int = 32000) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randperm(vocab, generator=g)[:count].sort().values


def forecast_inputs(L, H, n, steps, seed=41):
    """Seeded attention rows for the forecast fixture: causal prompt probabilities per layer, then one decode row
    per (step, layer) over all keys, peaked on a few drifting positions so that importance keeps changing."""
    rng = np.random.default_rng(seed)
    prompt = []
    for _ in range(L):
        s = rng.standard_normal((1, H, n, n)).astype(np.float32) * 2.0
        iu = np.triu_indices(n, 1)
        s[..., iu[0], iu[1]] = -np.inf
        p = np.exp(s - s.max(-1, keepdims=True))
        prompt.append((p / p.sum(-1, keepdims=True)).astype(np.float32))
    rows = []
    for t in range(steps):
        per_layer = []
        for _ in range(L):
            s = rng.standard_normal((1, H, 1, n + t + 1)).astype(np.float32)
            s[..., (7 * t) % (n + t)] += 4.0
            s[..., (3 * t + 11) % (n + t)] += 3.0
            p = np.exp(s - s.max(-1, keepdims=True))
            per_layer.append((p / p.sum(-1, keepdims=True)).astype(np.float32))
        rows.append(per_layer)
    return prompt, rows
