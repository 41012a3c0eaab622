"""Plain statement of the sampling kernel's arithmetic (mini_inference_b200/csrc/sampling.cu):
the integer hash in int64 with 32-bit masks, the Gumbel noise and the argmax."""
import torch

M32 = 0xFFFFFFFF


def fmix32(h):
    h = h ^ (h >> 16)
    h = (h * 0x85EBCA6B) & M32
    h = h ^ (h >> 13)
    h = (h * 0xC2B2AE35) & M32
    return h ^ (h >> 16)


def gumbel_noise(seed, counter, vocab, device="cpu"):
    i = torch.arange(vocab, dtype=torch.int64, device=device)
    h = fmix32(i ^ ((int(seed) * 0x9E3779B1) & M32))
    h = fmix32(h ^ ((int(counter) * 0x85EBCA77) & M32))
    u = ((h >> 8).to(torch.float32) + 0.5) * (1.0 / 16777216.0)
    return -torch.log(-torch.log(u))


def perturbed_scores(logits, temperatures, seeds, counters):
    """Row r: logits/T + gumbel when T > 0, else the logits."""
    rows = []
    for r in range(logits.shape[0]):
        t = float(temperatures[r])
        if t > 0:
            g = gumbel_noise(int(seeds[r]) & M32, int(counters[r]) & M32, logits.shape[1], logits.device)
            rows.append(logits[r].float() * (1.0 / max(t, 1e-5)) + g)
        else:
            rows.append(logits[r].float())
    return torch.stack(rows)


def gumbel_sample_reference(logits, temperatures, seeds, counters):
    if temperatures is None:
        return logits.argmax(-1).to(torch.int32)
    return perturbed_scores(logits, temperatures, seeds, counters).argmax(-1).to(torch.int32)
