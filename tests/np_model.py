"""An independent float64 numpy model of the Llama-2 decode step on dequantised weights, written
from the published llama2.c algorithm (not from the oracle's code), used to cross-check the oracle."""
import numpy as np

GROUP, GROUP_BYTES = 256, 264


def dequant(groups: np.ndarray, n: int) -> np.ndarray:
    g = np.ascontiguousarray(groups, dtype=np.uint8).reshape(-1, GROUP_BYTES)
    mn = g[:, 0:4].copy().view(">f4").astype(np.float64).reshape(-1, 1)
    mx = g[:, 4:8].copy().view(">f4").astype(np.float64).reshape(-1, 1)
    vals = g[:, 8:].astype(np.float64) * ((mx - mn) / 255.0) + mn
    return vals.reshape(-1)[:n]


class NumpyModel:
    def __init__(self, cfg, tensors):
        self.cfg = cfg
        d, h, L, kv = cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.dim * cfg.n_kv_heads // cfg.n_heads
        dq = lambda t, n: dequant(tensors[t], n)
        self.emb = np.asarray(tensors[0], dtype=np.float64).reshape(cfg.vocab_size, d)
        self.rms_att = dq(1, L * d).reshape(L, d)
        self.wq = dq(2, L * d * d).reshape(L, d, d)
        self.wk = dq(3, L * kv * d).reshape(L, kv, d)
        self.wv = dq(4, L * kv * d).reshape(L, kv, d)
        self.wo = dq(5, L * d * d).reshape(L, d, d)
        self.rms_ffn = dq(6, L * d).reshape(L, d)
        self.w1 = dq(7, L * h * d).reshape(L, h, d)
        self.w2 = dq(8, L * d * h).reshape(L, d, h)
        self.w3 = dq(9, L * h * d).reshape(L, h, d)
        self.rms_final = dq(10, d)
        self.wcls = self.emb if cfg.shared_classifier else np.asarray(tensors[11], dtype=np.float64).reshape(cfg.vocab_size, d)
        self.kc = np.zeros((L, cfg.seq_len, kv))
        self.vc = np.zeros((L, cfg.seq_len, kv))

    @staticmethod
    def _rms(x, w):
        return w * (x / np.sqrt(np.mean(x * x) + 1e-5))

    def forward(self, token, pos):
        c = self.cfg
        hs = c.dim // c.n_heads
        kv_mul = c.n_heads // c.n_kv_heads
        x = self.emb[token].copy()
        for l in range(c.n_layers):
            xb = self._rms(x, self.rms_att[l])
            q, k, v = self.wq[l] @ xb, self.wk[l] @ xb, self.wv[l] @ xb
            for vec in (q, k):
                for i in range(0, vec.size, 2):
                    freq = 1.0 / (10000.0 ** ((i % hs) / hs))
                    a = pos * freq
                    v0, v1 = vec[i], vec[i + 1]
                    vec[i] = v0 * np.cos(a) - v1 * np.sin(a)
                    vec[i + 1] = v0 * np.sin(a) + v1 * np.cos(a)
            self.kc[l, pos], self.vc[l, pos] = k, v
            out = np.zeros(c.dim)
            for h in range(c.n_heads):
                kvh = h // kv_mul
                ks = self.kc[l, :pos + 1, kvh * hs:(kvh + 1) * hs]
                vs = self.vc[l, :pos + 1, kvh * hs:(kvh + 1) * hs]
                s = ks @ q[h * hs:(h + 1) * hs] / np.sqrt(hs)
                p = np.exp(s - s.max())
                p /= p.sum()
                out[h * hs:(h + 1) * hs] = p @ vs
            x = x + self.wo[l] @ out
            xb = self._rms(x, self.rms_ffn[l])
            h1, h3 = self.w1[l] @ xb, self.w3[l] @ xb
            x = x + self.w2[l] @ (h1 / (1.0 + np.exp(-h1)) * h3)
        x = self._rms(x, self.rms_final)
        return self.wcls @ x
