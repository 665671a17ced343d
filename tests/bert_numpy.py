"""CPU restatement of the host runtime's BERT-base encoder (tacker_b200/host/dnn/models.cc Bert::Bert) for checking
the hidden states the `aker` binary computes.  Test infrastructure; conventions as in resnet50_numpy.py."""
import numpy as np

from resnet50_numpy import Net


def f16(x):
    return x.astype(np.float16).astype(np.float32)


def forward(oracle, layers=12, batch=8, seq=128):
    hidden, heads, dh, ffn, vocab = 768, 12, 64, 3072, 30522
    rows = batch * seq
    net = Net(oracle)
    tokens = (oracle.uniform_f32(rows, 77, 0.0, 1.0) * np.float32(vocab)).astype(np.uint64)
    x = np.empty((rows, hidden), np.float32)
    for r in range(rows):
        word = oracle.uniform_f32(hidden, 1000 + int(tokens[r]), 0.0, 1.0)
        pos = oracle.uniform_f32(hidden, 900000 + r % seq, 0.0, 1.0)
        x[r] = (word - np.float32(0.5)) * np.float32(0.1) + (pos - np.float32(0.5)) * np.float32(0.02)
    x = net.layernorm(x)
    split = lambda t: f16(t).reshape(batch, seq, heads, dh).transpose(0, 2, 1, 3)          # [B][heads][S][dh]
    for _ in range(layers):
        q, k, v = (net.dense(x, hidden, 0) for _ in range(3))
        net.next_id += 3                                                                   # the three head splits
        scores = np.matmul(split(q), split(k).transpose(0, 1, 3, 2)) * np.float32(1.0 / np.sqrt(np.float32(dh)))
        net.next_id += 2                                                                   # batched product, softmax
        e = np.exp(scores - scores.max(axis=-1, keepdims=True))
        p = (e / e.sum(axis=-1, keepdims=True)).astype(np.float32)
        net.next_id += 3                                                                   # fp16 copy, batched product, merge
        ctx = np.matmul(f16(p), split(v)).transpose(0, 2, 1, 3).reshape(rows, hidden).astype(np.float32)
        x = net.layernorm(net.add(net.dense(ctx, hidden, 0), x, 0))
        h = net.dense(net.dense(x, ffn, 2), hidden, 0)
        x = net.layernorm(net.add(h, x, 0))
    return x
