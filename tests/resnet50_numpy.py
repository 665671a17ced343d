"""CPU restatement of the host runtime's ResNet-50 (tacker_b200/host/dnn/models.cc Resnet50::Resnet50 and the
builders it uses) for checking the class scores the `aker` binary computes.  Test infrastructure.

Same seeded input and weights, same node numbering (it fixes the seeds), fp16-rounded GEMM operands with binary32
accumulation, fp32 activations, NHWC; see vgg16_numpy.py for the tolerance this is held to."""
import numpy as np

from vgg16_numpy import half_weights, normal_input, round_up


class Net:
    def __init__(self, oracle):
        self.oracle = oracle
        self.next_id = 0

    def conv(self, x, cout, k, pad, stride, act):
        H, W, C = x.shape
        conv_id = self.next_id
        self.next_id += 1
        K = k * k * C
        w = half_weights(self.oracle, round_up(cout, 64) * round_up(K, 64), 1000 + conv_id, np.sqrt(np.float32(6.0) / np.float32(K)))
        w = w.reshape(round_up(cout, 64), round_up(K, 64))[:cout, :K]       # k index = (i * k + j) * C + channel
        bias = self.oracle.uniform_f32(cout, 5000 + self.next_id, -0.05, 0.05)
        self.next_id += 1                                                   # the bias + activation node
        OH, OW = (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
        xp = np.zeros((H + 2 * pad, W + 2 * pad, C), np.float32)
        xp[pad:pad + H, pad:pad + W] = x.astype(np.float16).astype(np.float32)
        cols = np.concatenate([xp[i:i + stride * (OH - 1) + 1:stride, j:j + stride * (OW - 1) + 1:stride]
                               for i in range(k) for j in range(k)], axis=2).reshape(OH * OW, K)
        y = cols @ w.T + bias
        return (np.maximum(y, 0.0) if act else y).astype(np.float32).reshape(OH, OW, cout)

    def pool(self, x):
        H, W, C = x.shape
        self.next_id += 1
        return x[:2 * (H // 2), :2 * (W // 2)].reshape(H // 2, 2, W // 2, 2, C).max(axis=(1, 3))

    def add(self, a, b, act):
        self.next_id += 2 if act else 1                                     # the addition, then the activation node
        y = a + b
        return np.maximum(y, 0.0) if act else y

    def dense(self, x, out, act):
        dense_id = self.next_id
        self.next_id += 1
        K = x.shape[1]
        w = half_weights(self.oracle, round_up(out, 64) * round_up(K, 64), 2000 + dense_id, np.sqrt(np.float32(6.0) / np.float32(K)))
        w = w.reshape(round_up(out, 64), round_up(K, 64))[:out, :K]
        bias = self.oracle.uniform_f32(out, 6000 + self.next_id, -0.05, 0.05)
        self.next_id += 1
        y = x.astype(np.float16).astype(np.float32) @ w.T + bias
        if act == 1:
            y = np.maximum(y, 0.0)
        elif act == 2:                                                       # GELU, tanh form
            y = 0.5 * y * (1.0 + np.tanh(0.7978845608028654 * (y + 0.044715 * y * y * y)))
        return y.astype(np.float32)

    def layernorm(self, x):
        self.next_id += 1
        cols = x.shape[1]
        gamma = self.oracle.uniform_f32(cols, 7000 + self.next_id, 0.9, 1.1)
        beta = self.oracle.uniform_f32(cols, 7500 + self.next_id, -0.05, 0.05)
        mean = x.mean(axis=1, keepdims=True, dtype=np.float64)
        var = ((x - mean) ** 2).mean(axis=1, keepdims=True, dtype=np.float64)
        return (((x - mean) / np.sqrt(var + 1e-12)) * gamma + beta).astype(np.float32)


def forward(oracle, num_classes=1000):
    net = Net(oracle)
    x = normal_input(oracle, 224 * 224 * 3, 43).reshape(224, 224, 3)
    x = net.conv(x, 64, 7, 3, 2, 1)
    x = net.pool(x)
    for s, (nblocks, width) in enumerate(zip((3, 4, 6, 3), (64, 128, 256, 512))):
        for b in range(nblocks):
            stride = 2 if (b == 0 and s > 0) else 1
            shortcut = net.conv(x, 4 * width, 1, 0, stride, 0) if b == 0 else x
            y = net.conv(x, width, 1, 0, 1, 1)
            y = net.conv(y, width, 3, 1, stride, 1)
            y = net.conv(y, 4 * width, 1, 0, 1, 0)
            x = net.add(y, shortcut, 1)
    while x.shape[0] > 1:
        x = net.pool(x)
    return net.dense(x.reshape(1, -1), num_classes, 0)[0]
