"""ctypes wrappers of the host-side runners for the sequence head and the streaming agent
(include/aig_host.h: aig_seq_*, aig_agent_*).  Thin: every method is one C call."""
import ctypes

from . import (AIG_C3D_MAX_LAYERS, AIG_CNN_MAX_BLOCKS, ACT_SWISH, AigError, C3dConfig, CnnConfig, SeqConfig, c_int, c_void_p, lib, ptr)


def _device_copy(ctx, addr, shape, dtype):
    """Copy a device view owned by a runner into a fresh torch tensor."""
    import torch

    out = torch.empty(shape, dtype=dtype, device="cuda:%d" % ctx.device)
    ctx.call("aig_memcpy", c_void_p(out.data_ptr()), c_void_p(addr), out.numel() * out.element_size())
    ctx.sync()
    return out


def cnn_config(batch, height, width, widths=(32, 64, 128, 256, 256), k0=5, n_out=18, n_sigmoid=16, act=ACT_SWISH, slope=0.01):
    w = (c_int * (AIG_CNN_MAX_BLOCKS + 1))(*widths)
    return CnnConfig(batch, height, width, len(widths) - 1, w, k0, n_out, n_sigmoid, act, slope)


class SeqHead:
    def __init__(self, ctx, batch, seq_len, in_c=512, hidden=512, layers=2, heads=8, n_out=18, n_sigmoid=16, rope_base=10000.0,
                 window=0):
        self.ctx = ctx
        self.cfg = SeqConfig(batch, seq_len, in_c, hidden, layers, heads, n_out, n_sigmoid, rope_base, window)
        self.handle = c_void_p()
        rc = lib().aig_seq_create(ctx.handle, ctypes.byref(self.cfg), ctypes.byref(self.handle))
        if rc != 0:
            raise AigError(rc, lib().aig_last_error(ctx.handle).decode())

    def check(self, rc):
        if rc != 0:
            raise AigError(rc, lib().aig_seq_last_error(self.handle).decode())

    def param_bytes(self):
        return lib().aig_seq_param_bytes(ctypes.byref(self.cfg))

    def load_bytes(self, blob):
        buf = (ctypes.c_char * len(blob)).from_buffer_copy(blob)
        self.check(lib().aig_seq_load_memory(self.handle, ctypes.cast(buf, c_void_p), len(blob)))

    def forward(self, emb_bt, pos0=0):
        self.check(lib().aig_seq_forward(self.handle, ptr(emb_bt), pos0))

    def step(self, emb_t):
        self.check(lib().aig_seq_step(self.handle, ptr(emb_t)))

    def reset(self):
        self.check(lib().aig_seq_reset(self.handle))

    def outputs_f32(self, step=False):
        import torch

        c = self.cfg
        shape = (c.batch, c.n_out) if step else (c.batch, c.seq_len, c.n_out)
        return _device_copy(self.ctx, lib().aig_seq_outputs_f32(self.handle), shape, torch.float32)

    def lstm_output(self, step=False):
        import torch

        c = self.cfg
        shape = (c.batch, c.hidden) if step else (c.batch, c.seq_len, c.hidden)
        return _device_copy(self.ctx, lib().aig_seq_lstm_output(self.handle), shape, torch.float16)

    def close(self):
        if self.handle:
            lib().aig_seq_destroy(self.handle)
            self.handle = c_void_p()


class Agent:
    def __init__(self, ctx, batch, height, width, widths=(32, 64, 128, 256, 256), d=512, layers=2, heads=8, n_out=18, n_sigmoid=16,
                 rope_base=10000.0, window=64):
        self.ctx = ctx
        self.ccfg = cnn_config(batch, height, width, widths, n_out=n_out, n_sigmoid=n_sigmoid)
        self.scfg = SeqConfig(batch, window, d, d, layers, heads, n_out, n_sigmoid, rope_base, window)
        self.handle = c_void_p()
        rc = lib().aig_agent_create(ctx.handle, ctypes.byref(self.ccfg), ctypes.byref(self.scfg), ctypes.byref(self.handle))
        if rc != 0:
            raise AigError(rc, lib().aig_last_error(ctx.handle).decode())

    def check(self, rc):
        if rc != 0:
            raise AigError(rc, lib().aig_agent_last_error(self.handle).decode())

    def param_bytes(self):
        return lib().aig_agent_param_bytes(ctypes.byref(self.ccfg), ctypes.byref(self.scfg))

    def load_bytes(self, blob):
        buf = (ctypes.c_char * len(blob)).from_buffer_copy(blob)
        self.check(lib().aig_agent_load_memory(self.handle, ctypes.cast(buf, c_void_p), len(blob)))

    def step(self, bgra_dev):
        self.check(lib().aig_agent_step(self.handle, ptr(bgra_dev)))

    def step_host(self, bgra_host, out_host):
        self.check(lib().aig_agent_step_host(self.handle, ptr(bgra_host), ptr(out_host)))

    def reset(self):
        self.check(lib().aig_agent_reset(self.handle))

    def outputs_f32(self):
        import torch

        return _device_copy(self.ctx, lib().aig_agent_outputs_f32(self.handle), (self.scfg.batch, self.scfg.n_out), torch.float32)

    def close(self):
        if self.handle:
            lib().aig_agent_destroy(self.handle)
            self.handle = c_void_p()


class ClipEncoder:
    """Temporal clip encoder (aig_c3d_*): Conv3D+BN+LeakyReLU layers, 2x2 adaptive pool, FC head."""

    def __init__(self, ctx, batch, depth, height, width, widths=(3, 32, 64, 128), n_out=18, n_sigmoid=16, slope=0.01):
        self.ctx = ctx
        w = (c_int * (AIG_C3D_MAX_LAYERS + 1))(*widths)
        self.cfg = C3dConfig(batch, depth, height, width, len(widths) - 1, w, n_out, n_sigmoid, slope)
        self.handle = c_void_p()
        rc = lib().aig_c3d_create(ctx.handle, ctypes.byref(self.cfg), ctypes.byref(self.handle))
        if rc != 0:
            raise AigError(rc, lib().aig_last_error(ctx.handle).decode())

    def check(self, rc):
        if rc != 0:
            raise AigError(rc, lib().aig_c3d_last_error(self.handle).decode())

    def param_bytes(self):
        return lib().aig_c3d_param_bytes(ctypes.byref(self.cfg))

    def load_bytes(self, blob):
        buf = (ctypes.c_char * len(blob)).from_buffer_copy(blob)
        self.check(lib().aig_c3d_load_memory(self.handle, ctypes.cast(buf, c_void_p), len(blob)))

    def forward(self, clips_dev):
        self.check(lib().aig_c3d_forward(self.handle, ptr(clips_dev)))

    def outputs_f32(self):
        import torch

        return _device_copy(self.ctx, lib().aig_c3d_outputs_f32(self.handle), (self.cfg.batch, self.cfg.n_out), torch.float32)

    def features(self):
        import torch

        feat = self.cfg.widths[self.cfg.n_layers] * 4
        return _device_copy(self.ctx, lib().aig_c3d_features(self.handle), (self.cfg.batch, feat), torch.float16)

    def close(self):
        if self.handle:
            lib().aig_c3d_destroy(self.handle)
            self.handle = c_void_p()
