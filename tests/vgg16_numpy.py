"""CPU restatement of the host runtime's VGG16 (tacker_b200/host/dnn/models.cc VGG16::VGG16 and the builders it
uses) for checking the logits the `aker` binary computes.  Test infrastructure.

Same seeded input and weights (the counter generator of tacker_b200/host/util.h, which is the oracle's), same layer
numbering, fp16-rounded GEMM operands with binary32 accumulation, fp32 activations, NHWC.  The accumulation order
inside a dot product differs from the tensor cores', so the comparison is held to 1e-2 of the largest score."""
import numpy as np


def unit_draws(oracle, seed, n):
    return oracle.uniform_f32(n, seed, 0.0, 1.0)


def normal_input(oracle, n, seed):
    u = unit_draws(oracle, seed, 2 * n)
    u1 = u[0::2] + np.float32(2.98e-8)
    u2 = u[1::2]
    return (np.sqrt(np.float32(-2.0) * np.log(u1)) * np.cos(np.float32(6.2831853) * u2)).astype(np.float32)


def half_weights(oracle, count, seed, scale):
    w = (unit_draws(oracle, seed, count) * np.float32(2.0) - np.float32(1.0)) * np.float32(scale)
    return w.astype(np.float16).astype(np.float32)


def round_up(v, m):
    return (v + m - 1) // m * m


def forward(oracle, num_classes=1000):
    H = W = 224
    C = 3
    x = normal_input(oracle, H * W * C, 42).reshape(H, W, C)
    next_id = 0
    cfg = [64, 64, -1, 128, 128, -1, 256, 256, 256, -1, 512, 512, 512, -1, 512, 512, 512, -1]
    for c in cfg:
        if c < 0:
            next_id += 1                                     # the pooling node
            x = x.reshape(H // 2, 2, W // 2, 2, C).max(axis=(1, 3))
            H //= 2
            W //= 2
            continue
        conv_id = next_id
        next_id += 1
        K = 9 * C
        K_pad, N_pad = round_up(K, 64), round_up(c, 64)
        w = half_weights(oracle, N_pad * K_pad, 1000 + conv_id, np.sqrt(np.float32(6.0) / np.float32(K)))
        w = w.reshape(N_pad, K_pad)[:c, :K]                  # k = (i * 3 + j) * C + channel
        bias = oracle.uniform_f32(c, 5000 + next_id, -0.05, 0.05)
        next_id += 1                                         # the bias + activation node
        xh = x.astype(np.float16).astype(np.float32)
        xp = np.zeros((H + 2, W + 2, C), np.float32)
        xp[1:-1, 1:-1] = xh
        cols = np.concatenate([xp[i:i + H, j:j + W] for i in range(3) for j in range(3)], axis=2).reshape(H * W, K)
        y = cols @ w.T + bias
        x = np.maximum(y, 0.0).astype(np.float32).reshape(H, W, c)
        C = c
    x = x.reshape(1, H * W * C)
    for out, act in ((4096, 1), (4096, 1), (num_classes, 0)):
        dense_id = next_id
        next_id += 1
        K = x.shape[1]
        K_pad, N_pad = round_up(K, 64), round_up(out, 64)
        w = half_weights(oracle, N_pad * K_pad, 2000 + dense_id, np.sqrt(np.float32(6.0) / np.float32(K)))
        w = w.reshape(N_pad, K_pad)[:out, :K]
        bias = oracle.uniform_f32(out, 6000 + next_id, -0.05, 0.05)
        next_id += 1
        y = x.astype(np.float16).astype(np.float32) @ w.T + bias
        x = (np.maximum(y, 0.0) if act else y).astype(np.float32)
    scores = x[0]
    e = np.exp(scores - scores.max())
    return scores, (e / e.sum()).astype(np.float32)
