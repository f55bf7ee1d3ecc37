"""Model and KV-cache objects over the native library (new API, in the style of Kernel).

Model configs of the benchmark are in CONFIGS; `Model(ctx, cfg)` allocates the weights on the
context's device (this rank's shard under tensor parallelism), `init_random(seed)` fills them
from the seeded generator, `new_cache(batch, maxlen)` creates the KV cache object.
"""
import ctypes as C

import numpy as np

from . import native as N

GPT2, QWEN3 = 0, 1

CONFIGS = {
    # GPT-2 small: 12 layers, d 768, 12 heads x 64, MLP 3072, LN eps 1e-5, 1024 positions, tied
    "gpt2-small": dict(arch=GPT2, n_layers=12, d_model=768, n_q_heads=12, n_kv_heads=12, head_dim=64, d_ff=3072,
                       vocab=50257, max_pos=1024, tied=1, eps=1e-5, rope_theta=0.0),
    # Qwen3-0.6B: 28 layers, hidden 1024, 16 Q / 8 KV heads x 128, MLP 3072, eps 1e-6, theta 1e6, tied
    "qwen3-0.6b": dict(arch=QWEN3, n_layers=28, d_model=1024, n_q_heads=16, n_kv_heads=8, head_dim=128, d_ff=3072,
                       vocab=151936, max_pos=4096, tied=1, eps=1e-6, rope_theta=1e6),
    # Qwen3-8B: 36 layers, hidden 4096, 32 Q / 8 KV heads x 128, MLP 12288, untied head
    "qwen3-8b": dict(arch=QWEN3, n_layers=36, d_model=4096, n_q_heads=32, n_kv_heads=8, head_dim=128, d_ff=12288,
                     vocab=151936, max_pos=4096, tied=0, eps=1e-6, rope_theta=1e6),
}


def make_config(cfg):
    c = N.ModelConfig()
    for k in ("arch", "n_layers", "d_model", "n_q_heads", "n_kv_heads", "head_dim", "d_ff", "vocab", "max_pos", "tied"):
        setattr(c, k, int(cfg[k]))
    c.eps = float(cfg["eps"])
    c.rope_theta = float(cfg["rope_theta"])
    return c


class Model:
    def __init__(self, ctx, cfg):
        self.ctx, self.cfg = ctx, dict(cfg)
        self.h = C.c_void_p()
        c = make_config(cfg)
        N.check(N.lib().strictb200_model_create(ctx.h, C.byref(c), C.byref(self.h)))

    def init_random(self, seed):
        N.check(N.lib().strictb200_model_init_random(self.h, seed))
        return self

    def set_tensor(self, name, host):
        host = np.ascontiguousarray(host)
        N.check(N.lib().strictb200_model_set_tensor(self.h, name.encode(), N.ptr(host), host.nbytes))

    def get_tensor(self, name, dtype, count):
        out = np.empty(count, dtype)
        N.check(N.lib().strictb200_model_get_tensor(self.h, name.encode(), N.ptr(out), out.nbytes))
        return out

    def weight_bytes(self):
        n = C.c_uint64()
        N.check(N.lib().strictb200_model_weight_bytes(self.h, C.byref(n)))
        return n.value

    def set_graph(self, enabled):
        N.check(N.lib().strictb200_model_set_graph(self.h, 1 if enabled else 0))

    def new_cache(self, batch, maxlen):
        return KvCache(self, batch, maxlen)

    def dispose(self):
        if self.h:
            N.lib().strictb200_model_destroy(self.h)
            self.h = C.c_void_p()

    Dispose = dispose


class KvCache:
    def __init__(self, model, batch, maxlen):
        self.model, self.B = model, batch
        self.h = C.c_void_p()
        N.check(N.lib().strictb200_kv_create(model.h, batch, maxlen, C.byref(self.h)))

    def reset(self):
        N.check(N.lib().strictb200_kv_reset(self.h))

    def lens(self):
        out = np.empty(self.B, np.int32)
        N.check(N.lib().strictb200_kv_lens(self.h, N.ptr(out)))
        return out

    def fill_synthetic(self, seed, length):
        N.check(N.lib().strictb200_kv_fill_synthetic(self.h, seed, length))

    def prefill(self, tokens, lens=None, want_logits=False):
        """tokens [B,S] int32; returns (next_ids[B], logits[B,V] or None)."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        B, S = tokens.shape
        lens = np.full(B, S, np.int32) if lens is None else np.ascontiguousarray(lens, dtype=np.int32)
        nxt = np.empty(B, np.int32)
        logits = np.empty((B, self.model.cfg["vocab"]), np.float32) if want_logits else None
        N.check(N.lib().strictb200_prefill(self.model.h, self.h, N.ptr(tokens), N.ptr(lens), B, S, N.ptr(nxt), N.ptr(logits)))
        return nxt, logits

    def decode_step(self, ids, want_logits=False, out=None):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        nxt = np.empty(self.B, np.int32) if out is None else out
        logits = np.empty((self.B, self.model.cfg["vocab"]), np.float32) if want_logits else None
        N.check(N.lib().strictb200_decode_step(self.model.h, self.h, N.ptr(ids), N.ptr(nxt), N.ptr(logits)))
        return nxt, logits

    def generate(self, ids, n_steps):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        out = np.empty((n_steps, self.B), np.int32)
        N.check(N.lib().strictb200_generate(self.model.h, self.h, N.ptr(ids), n_steps, N.ptr(out)))
        return out

    def decode_steps_device(self, n_steps):
        """n greedy steps with ids resident on the device (no host copies, asynchronous)."""
        N.check(N.lib().strictb200_decode_steps_device(self.model.h, self.h, None, n_steps))

    KERNEL_CLASSES = ("embed", "gemm_qkv", "rope_kvappend", "attn_decode", "gemm_o", "rownorm", "gemm_gate_up", "swiglu",
                      "gemm_down", "head", "allreduce", "attn_merge")

    def profile_decode(self, n_steps):
        """Per-kernel-class device time of n plain-launch decode steps: {class: (total_ms, calls)}."""
        ms = np.zeros(len(self.KERNEL_CLASSES), np.float32)
        calls = np.zeros(len(self.KERNEL_CLASSES), np.uint64)
        N.check(N.lib().strictb200_profile_decode(self.model.h, self.h, n_steps, N.ptr(ms), N.ptr(calls), len(ms)))
        return {k: (float(ms[i]), int(calls[i])) for i, k in enumerate(self.KERNEL_CLASSES)}

    def decode_bytes(self):
        n = C.c_uint64()
        N.check(N.lib().strictb200_decode_bytes(self.model.h, self.h, C.byref(n)))
        return n.value

    def dispose(self):
        if self.h:
            N.lib().strictb200_kv_destroy(self.h)
            self.h = C.c_void_p()

    Dispose = dispose
