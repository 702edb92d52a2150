"""Python binding of the B200 C ABI (include/aig_b200.h) for tests and benchmarks.

The product is the shared library ``libaig_b200.so`` built from ``csrc/`` and ``host/``; this module
only loads it with ctypes, declares every entry point's signature, and offers thin helpers that take
torch CUDA tensors (torch is used for device memory and streams, nothing else).  There is no
fallback: if the library is missing or a call fails, an exception is raised.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libaig_b200.so")

c_int, c_float, c_size_t, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_size_t, ctypes.c_void_p
P = c_void_p
PP = ctypes.POINTER(c_void_p)
PI = ctypes.POINTER(c_int)

ACT_NONE, ACT_RELU, ACT_SWISH, ACT_LEAKY = 0, 1, 2, 3


class ConvDesc(ctypes.Structure):
    _fields_ = [(n, c_int) for n in ("batch", "in_c", "in_d", "in_h", "in_w", "out_c", "kd", "kh", "kw", "sd", "sh",
                                     "sw", "pd", "ph", "pw", "act")] + [("slope", c_float), ("two_step", c_int)]


# name -> argtypes (restype is int unless listed in _RESTYPES)
SIGNATURES = {
    "aig_ctx_create": [PP, c_int],
    "aig_ctx_destroy": [P],
    "aig_ctx_set_stream": [P, P],
    "aig_ctx_stream": [P],
    "aig_ctx_sync": [P],
    "aig_last_error": [P],
    "aig_selftest_expiring_wait": [P, ctypes.c_longlong],
    "aig_device_sm_count": [P],
    "aig_memcpy": [P, P, P, c_size_t],
    "aig_graph_begin": [P],
    "aig_graph_end": [P, PP],
    "aig_graph_launch": [P, P],
    "aig_graph_destroy": [P],
    "aig_bgra_to_planar": [P, P, P, c_int],
    "aig_convert_normalize": [P, P, P, c_size_t],
    "aig_preprocess_bgra": [P, P, P, c_int, c_int],
    "aig_unconvert_unnormalize": [P, P, P, c_size_t],
    "aig_half_to_float": [P, P, P, c_size_t],
    "aig_resize_box": [P, P, c_int, P, P, c_int, c_int, c_int, c_int, c_int, c_int],
    "aig_mse_loss2": [P, P, P, c_int, c_int, c_int, ctypes.POINTER(c_float), ctypes.POINTER(c_float)],
    "aig_loss_gradient": [P, P, P, P, ctypes.c_longlong],
    "aig_any_nan_half": [P, P, ctypes.c_longlong, ctypes.POINTER(c_int)],
    "aig_swish_backward": [P, P, P, ctypes.c_longlong],
    "aig_leaky_relu_backward": [P, P, P, ctypes.c_longlong, c_float],
    "aig_sigmoid_backward": [P, P, P, c_int, c_int, ctypes.c_longlong],
    "aig_bias_gradient": [P, P, P, c_int, c_int],
    "aig_sgd_step_f16": [P, P, P, ctypes.c_longlong, c_float, c_float],
    "aig_sgd_step_f32": [P, P, P, ctypes.c_longlong, c_float, c_float],
    "aig_adamw_step_f32": [P, P, P, P, P, ctypes.c_longlong, c_float, c_int, c_float],
    "aig_adamw_step_f16": [P, P, P, P, P, ctypes.c_longlong, c_float, c_int, c_float],
    "aig_fc_backward_plan_create": [P, c_int, c_int, c_int, P],
    "aig_fc_backward": [P, P, P, P, P, P, P],
    "aig_fc_backward_plan_destroy": [P],
    "aig_fc_backward_weight_storage": [P],
    "aig_fc_adamw_update": [P, P, c_int, c_int, P, P, P, P, P, P, P, P, c_float, c_int, c_float],
    "aig_process_output": [P, P, P, c_int],
    "aig_process_output_to": [P, P, P, P],
    "aig_float_to_half": [P, P, P, c_size_t],
    "aig_nchw_to_nhwc": [P, P, P, c_int, c_int, c_int],
    "aig_nhwc_to_nchw": [P, P, P, c_int, c_int, c_int],
    "aig_leaky_relu_forward": [P, P, c_int, c_float],
    "aig_swish_forward": [P, P, c_int],
    "aig_relu_forward": [P, P, c_int],
    "aig_sigmoid_forward": [P, P, c_int, c_int, c_int],
    "aig_tanh_tail_forward": [P, P, c_int, c_int, c_int],
    "aig_add_forward": [P, P, P, c_int],
    "aig_batchnorm_forward": [P, P, P, P, P, P, P, c_int, c_int, c_int, c_float, c_int],
    "aig_layernorm_forward": [P, P, P, P, P, P, P, c_int, c_int, c_int, c_float],
    "aig_layernorm_rows_forward": [P, P, P, P, P, c_int, c_int, c_float],
    "aig_spatial_attention_forward": [P] * 10 + [c_int] * 6,
    "aig_spatial_mask_forward": [P, P, P, c_float, P, c_int, c_int, c_int],
    "aig_global_avgpool_nhwc": [P, P, P, c_int, c_int, c_int],
    "aig_adaptive_avgpool3d_ndhwc": [P, P, P] + [c_int] * 7,
    "aig_fc_head_forward": [P, P, P, P, P, P, c_int, c_int, c_int, c_int],
    "aig_cnn_head_forward": [P, P, P, c_float, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int],
    "aig_conv_plan_create": [P, ctypes.POINTER(ConvDesc), PP],
    "aig_conv_plan_destroy": [P],
    "aig_conv_plan_out_dims": [P, PI, PI, PI],
    "aig_conv_plan_set_weights": [P, P, P, P, P, P, P, c_float],
    "aig_conv_forward": [P, P, P, P],
    "aig_fc_plan_create": [P, c_int, c_int, c_int, c_int, c_float, c_int, PP],
    "aig_fc_plan_set_weights": [P, P, P, P, P, P, P, c_float],
    "aig_fc_plan_set_weights_out_in": [P, P, P],
    "aig_fc_plan_set_output_f32": [P, c_int],
    "aig_fc_plan_add_bias": [P, P],
    "aig_lstm_weight_count": [c_int, c_int, c_int, c_int],
    "aig_lstm_plan_create": [P, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, PP],
    "aig_lstm_plan_destroy": [P],
    "aig_lstm_plan_set_weights": [P, P],
    "aig_lstm_forward": [P, P, P, P, P, c_int],
    "aig_lstm_forward_noalloc": [P, P, P, P, c_int, c_int, c_int, c_int, c_float, c_int],
    "aig_mha_plan_create": [P, c_int, c_int, c_int, c_int, c_float, c_int, PP],
    "aig_mha_plan_destroy": [P],
    "aig_mha_plan_set_weights": [P, P, P, P, P],
    "aig_mha_forward": [P, P, P, c_int],
    "aig_mha_step": [P, P, P, c_int],
    "aig_mha_reset": [P],
    "aig_conv0_plan_create": [P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, PP],
    "aig_conv0_plan_create_3d": [P] + [c_int] * 12 + [c_float, PP],
    "aig_conv0_plan_destroy": [P],
    "aig_conv0_plan_out_dims": [P, PI, PI, PI],
    "aig_conv0_plan_set_weights": [P, P, P, P, P, P, P, c_float],
    "aig_conv0_forward_bgra": [P, P, P],
    "aig_conv0_forward_nchw": [P, P, P],
    "aig_conv0_forward_rgb_planar": [P, P, P],
    "aig_s2d_elems": [c_int, c_int, c_int, c_int],
    "aig_nhwc_to_s2d": [P, P, P, c_int, c_int, c_int, c_int],
    "aig_s2d_to_nhwc": [P, P, P, c_int, c_int, c_int, c_int],
    "aig_conv_plan_set_output_s2d": [P, c_int],
    "aig_conv0_plan_set_output_s2d": [P, c_int],
    "aig_resdown_plan_create": [P, c_int, c_int, c_int, c_int, c_int, c_int, c_float, PP],
    "aig_resdown_plan_set_weights": [P, P, P, P, P, P, P, c_float, P, P],
    "aig_resdown_forward": [P, P, P, P],
    "aig_conv_padded_rows": [c_int, c_int, c_int, c_int],
    "aig_resdown_plan_set_output_padded": [P, c_int],
    "aig_conv_plan_set_input_padded": [P, c_int],
    "aig_actions_from_outputs": [P, P, c_int, c_int, c_int],
    # include/aig_compat.h: the reference's launcher names (no context argument; most return void)
    "InitCUDA": [],
    "ConvertAndNormalize": [P, P, c_size_t],
    "UnConvertAndUnNormalize": [P, P, c_size_t],
    "ConvertFloatToHalf": [P, P, c_size_t],
    "ConvertHalfToFloat": [P, P, c_size_t],
    "HeInit": [P, c_int, c_float],
    "LeakyReluForward": [P, c_int, c_float],
    "SwishForward": [P, c_int],
    "SigmoidForward": [P, c_int, c_int, c_int],
    "LayerNormForward": [P, P, P, P, P, P, c_int, c_int, c_int],
    "SpatialAttentionForward": [P] * 9 + [c_int] * 5,
    "ARGBtoRGB": [P, P, c_int],
    "ARGBtoRGBplanar": [P, P, c_int],
    "aig_compat_context": [],
    "aig_compat_last_status": [],
    "aig_compat_set_attention_group": [c_int],
}
AIG_CNN_MAX_BLOCKS = 7


class CnnConfig(ctypes.Structure):
    _fields_ = [("batch", c_int), ("height", c_int), ("width", c_int), ("n_blocks", c_int),
                ("widths", c_int * (AIG_CNN_MAX_BLOCKS + 1)), ("k0", c_int), ("n_out", c_int), ("n_sigmoid", c_int),
                ("act", c_int), ("slope", c_float)]


SIGNATURES.update({
    "aig_cnn_create": [P, ctypes.POINTER(CnnConfig), PP],
    "aig_cnn_destroy": [P],
    "aig_cnn_last_error": [P],
    "aig_cnn_checkpoint_bytes": [ctypes.POINTER(CnnConfig)],
    "aig_cnn_load_memory": [P, P, c_size_t],
    "aig_cnn_load_file": [P, ctypes.c_char_p],
    "aig_cnn_forward": [P, P],
    "aig_cnn_forward_graph": [P, P],
    "aig_cnn_forward_rgb": [P, P],
    "aig_cnn_forward_graph_rgb": [P, P],
    "aig_cnn_submit_host_rgb": [P, c_int, P, P],
    "aig_cnn_infer_host": [P, P, P],
    "aig_cnn_submit_host": [P, c_int, P, P],
    "aig_cnn_wait": [P, c_int],
    "aig_cnn_outputs_half": [P],
    "aig_cnn_outputs_f32": [P],
    "aig_cnn_features": [P],
    "aig_cnn_stage_output": [P, c_int, PI, PI, PI],
    "aig_cnn_kernel_launches": [P],
    "aig_cnn_profile_begin": [P, c_int],
    "aig_cnn_profile_end": [P, ctypes.POINTER(ctypes.c_double), c_int, PI],
    "aig_cnn_site_count": [P],
    "aig_cnn_site_name": [P, c_int],
    "aig_cnn_site_flops": [P, c_int],
    "aig_cnn_site_bytes": [P, c_int],
})


class SeqConfig(ctypes.Structure):
    _fields_ = [("batch", c_int), ("seq_len", c_int), ("in_c", c_int), ("hidden", c_int), ("layers", c_int), ("heads", c_int),
                ("n_out", c_int), ("n_sigmoid", c_int), ("rope_base", c_float), ("window", c_int)]


SIGNATURES.update({
    "aig_seq_create": [P, ctypes.POINTER(SeqConfig), PP],
    "aig_seq_destroy": [P],
    "aig_seq_last_error": [P],
    "aig_seq_param_bytes": [ctypes.POINTER(SeqConfig)],
    "aig_seq_load_memory": [P, P, c_size_t],
    "aig_seq_forward": [P, P, c_int],
    "aig_seq_step": [P, P],
    "aig_seq_reset": [P],
    "aig_seq_outputs_half": [P],
    "aig_seq_outputs_f32": [P],
    "aig_seq_lstm_output": [P],
    "aig_agent_create": [P, ctypes.POINTER(CnnConfig), ctypes.POINTER(SeqConfig), PP],
    "aig_agent_destroy": [P],
    "aig_agent_last_error": [P],
    "aig_agent_param_bytes": [ctypes.POINTER(CnnConfig), ctypes.POINTER(SeqConfig)],
    "aig_agent_load_memory": [P, P, c_size_t],
    "aig_agent_step": [P, P],
    "aig_agent_step_host": [P, P, P],
    "aig_agent_reset": [P],
    "aig_agent_outputs_f32": [P],
    "aig_refnn_create": [P, c_int, c_int, ctypes.c_char_p, PP],
    "aig_refnn_forward": [P, P, PP],
    "aig_refnn_input_size": [P, PI, PI],
    "aig_compat_handle_create": [PP],
    "aig_refnn_infer_frame": [P, P, P, P, P, P],
    "aig_refnn_destroy": [P],
    "aig_layers_last_error": [],
    "aig_layer_create": [P, ctypes.c_char_p, PI, c_int, PP],
    "aig_layer_forward": [P, P, PP],
    "aig_layer_backward": [P, P, PP],
    "aig_layer_update": [P, c_float],
    "aig_layer_load_file": [P, ctypes.c_char_p],
    "aig_layer_save_file": [P, ctypes.c_char_p],
    "aig_layer_param_bytes": [P],
    "aig_layer_out_count": [P],
    "aig_layer_destroy": [P],
})
SIGNATURES.update({
    "aig_recording_open": [ctypes.c_char_p, PP],
    "aig_recording_close": [P],
    "aig_recording_last_error": [P],
    "aig_recording_info": [P, PI, PI, ctypes.POINTER(ctypes.c_longlong)],
    "aig_recording_read": [P, ctypes.c_longlong, c_int, P, P, P],
    "aig_recording_targets": [P, P, c_int, P],
    "aig_cnn_infer_recording": [P, P, ctypes.c_longlong, ctypes.c_longlong, c_int, c_int, P],
})
AIG_C3D_MAX_LAYERS = 6


class C3dConfig(ctypes.Structure):
    _fields_ = [("batch", c_int), ("depth", c_int), ("height", c_int), ("width", c_int), ("n_layers", c_int),
                ("widths", c_int * (AIG_C3D_MAX_LAYERS + 1)), ("n_out", c_int), ("n_sigmoid", c_int), ("slope", c_float)]


SIGNATURES.update({
    "aig_c3d_create": [P, ctypes.POINTER(C3dConfig), PP],
    "aig_c3d_destroy": [P],
    "aig_c3d_last_error": [P],
    "aig_c3d_param_bytes": [ctypes.POINTER(C3dConfig)],
    "aig_c3d_load_memory": [P, P, c_size_t],
    "aig_c3d_forward": [P, P],
    "aig_c3d_outputs_f32": [P],
    "aig_c3d_features": [P],
})
_RESTYPES = {"aig_compat_context": c_void_p, "aig_fc_backward_weight_storage": c_void_p, "aig_recording_last_error": ctypes.c_char_p, "aig_layer_param_bytes": c_size_t, "aig_s2d_elems": c_size_t, "aig_conv_padded_rows": ctypes.c_longlong, "aig_c3d_last_error": ctypes.c_char_p, "aig_c3d_param_bytes": c_size_t, "aig_c3d_outputs_f32": c_void_p,
             "aig_c3d_features": c_void_p, "aig_ctx_stream": c_void_p, "aig_last_error": ctypes.c_char_p, "aig_cnn_last_error": ctypes.c_char_p,
             "aig_cnn_checkpoint_bytes": c_size_t, "aig_cnn_outputs_half": c_void_p, "aig_cnn_outputs_f32": c_void_p,
             "aig_cnn_features": c_void_p, "aig_cnn_stage_output": c_void_p, "aig_cnn_site_name": ctypes.c_char_p,
             "aig_cnn_site_flops": ctypes.c_double, "aig_cnn_site_bytes": ctypes.c_double,
             "aig_lstm_weight_count": c_size_t, "aig_seq_last_error": ctypes.c_char_p, "aig_seq_param_bytes": c_size_t,
             "aig_seq_outputs_half": c_void_p, "aig_seq_outputs_f32": c_void_p, "aig_seq_lstm_output": c_void_p,
             "aig_layers_last_error": ctypes.c_char_p, "aig_agent_last_error": ctypes.c_char_p, "aig_agent_param_bytes": c_size_t, "aig_agent_outputs_f32": c_void_p}

_lib = None


class AigError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("aig_b200 error %d: %s" % (code, msg))
        self.code = code


def lib():
    """Load libaig_b200.so (fails loudly when it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "libaig_b200.so is missing: build it with `python ai-gamer_b200/build.py` "
                "(there is no fallback implementation)")
        _lib = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.argtypes = args
            fn.restype = _RESTYPES.get(name, c_int)
    return _lib


def ptr(t):
    """Device (or host) address of a torch tensor / numpy array / None."""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        return c_void_p(t.data_ptr())
    return c_void_p(t.ctypes.data)


class Context:
    """One device + one stream (aig_ctx).  By default it adopts torch's current CUDA stream so that
    calls interleave correctly with torch allocations and copies."""

    def __init__(self, device=0, use_torch_stream=True):
        self.handle = c_void_p()
        rc = lib().aig_ctx_create(ctypes.byref(self.handle), device)
        if rc != 0:
            raise AigError(rc, lib().aig_last_error(None).decode())
        self.device = device
        if use_torch_stream:
            import torch

            if torch.cuda.current_stream(device).cuda_stream == 0:
                # the legacy default stream cannot be captured into a CUDA graph: switch torch (and this
                # context) to a fresh stream; work already queued on the default stream is waited for
                s = torch.cuda.Stream(device)
                s.wait_stream(torch.cuda.current_stream(device))
                torch.cuda.set_stream(s)
                self._torch_stream = s
            self.set_stream(torch.cuda.current_stream(device).cuda_stream)

    def check(self, rc):
        if rc != 0:
            raise AigError(rc, lib().aig_last_error(self.handle).decode())

    def call(self, name, *args):
        self.check(getattr(lib(), name)(self.handle, *args))

    def set_stream(self, cuda_stream):
        self.check(lib().aig_ctx_set_stream(self.handle, c_void_p(cuda_stream)))

    def sync(self):
        self.check(lib().aig_ctx_sync(self.handle))

    @property
    def sm_count(self):
        return lib().aig_device_sm_count(self.handle)

    def close(self):
        if self.handle:
            lib().aig_ctx_destroy(self.handle)
            self.handle = c_void_p()

    # -- CUDA graph of the frame loop
    def graph_begin(self):
        self.check(lib().aig_graph_begin(self.handle))

    def graph_end(self):
        g = c_void_p()
        self.check(lib().aig_graph_end(self.handle, ctypes.byref(g)))
        return g

    def graph_launch(self, g):
        self.check(lib().aig_graph_launch(self.handle, g))


class _Plan:
    _destroy = None

    def __init__(self, ctx):
        self.ctx = ctx
        self.handle = c_void_p()
        self._keep = []

    def check(self, rc):
        self.ctx.check(rc)

    def close(self):
        if self.handle:
            getattr(lib(), self._destroy)(self.handle)
            self.handle = c_void_p()

    def out_dims(self):
        d, h, w = c_int(), c_int(), c_int()
        getattr(lib(), self._dims)(self.handle, ctypes.byref(d), ctypes.byref(h), ctypes.byref(w))
        return d.value, h.value, w.value


def padded_rows(batch, h, w, pad=1):
    """Rows of a [batch][h][w][c] tensor in the padded position layout (aig_conv_padded_rows)."""
    return int(lib().aig_conv_padded_rows(batch, h, w, pad))


class ConvPlan(_Plan):
    """aig_conv_plan: tcgen05 implicit-GEMM convolution on channels-last tensors."""
    _destroy = "aig_conv_plan_destroy"
    _dims = "aig_conv_plan_out_dims"

    def __init__(self, ctx, batch, in_c, in_h, in_w, out_c, k, stride, pad, act=ACT_NONE, slope=0.01, two_step=False,
                 in_d=1, kd=1, sd=1, pd=0):
        super().__init__(ctx)
        self.desc = ConvDesc(batch, in_c, in_d, in_h, in_w, out_c, kd, k, k, sd, stride, stride, pd, pad, pad, act, slope,
                             1 if two_step else 0)
        self.check(lib().aig_conv_plan_create(ctx.handle, ctypes.byref(self.desc), ctypes.byref(self.handle)))

    def set_weights(self, w, bias, bn=None, eps=1e-6):
        g, b, m, v = bn if bn is not None else (None, None, None, None)
        self._keep = [w, bias, g, b, m, v]
        self.check(lib().aig_conv_plan_set_weights(self.handle, ptr(w), ptr(bias), ptr(g), ptr(b), ptr(m), ptr(v), eps))

    def forward(self, x, y, residual=None):
        self.check(lib().aig_conv_forward(self.handle, ptr(x), ptr(residual), ptr(y)))
        return y

    def set_input_padded(self, enable=True):
        """x and residual of forward() in the padded position layout (see padded_rows)."""
        self.check(lib().aig_conv_plan_set_input_padded(self.handle, 1 if enable else 0))



class ResDownPlan(_Plan):
    """aig_resdown_plan: main k4 s2 p1 conv (+BN+act) and k2 s2 p0 shortcut of a residual block as one launch
    over the space-to-depth view of the input."""
    _destroy = "aig_conv_plan_destroy"
    _dims = "aig_conv_plan_out_dims"

    def __init__(self, ctx, batch, in_c, in_h, in_w, out_c, act=ACT_NONE, slope=0.01):
        super().__init__(ctx)
        self.check(lib().aig_resdown_plan_create(ctx.handle, batch, in_c, in_h, in_w, out_c, act, slope, ctypes.byref(self.handle)))

    def set_weights(self, w_main, b_main, bn, w_short, b_short, eps=1e-6):
        g, b, m, v = bn if bn is not None else (None, None, None, None)
        self.check(lib().aig_resdown_plan_set_weights(self.handle, ptr(w_main), ptr(b_main), ptr(g), ptr(b), ptr(m), ptr(v), eps,
                                                      ptr(w_short), ptr(b_short)))

    def forward(self, x_s2d, y_main, y_short):
        self.check(lib().aig_resdown_forward(self.handle, ptr(x_s2d), ptr(y_main), ptr(y_short)))

    def set_output_padded(self, enable=True):
        """y_main / y_short in the padded position layout (rows: padded_rows(batch, Ho, Wo, 1))."""
        self.check(lib().aig_resdown_plan_set_output_padded(self.handle, 1 if enable else 0))


class FcPlan(_Plan):
    """aig_fc_plan_*: the same kernel as ConvPlan on a [rows][in_c] matrix."""
    _destroy = "aig_conv_plan_destroy"
    _dims = "aig_conv_plan_out_dims"

    def __init__(self, ctx, rows, in_c, out_c, act=ACT_NONE, slope=0.01, two_step=False):
        super().__init__(ctx)
        self.check(lib().aig_fc_plan_create(ctx.handle, rows, in_c, out_c, act, slope, 1 if two_step else 0,
                                            ctypes.byref(self.handle)))

    def set_weights(self, w_in_out, bias, bn=None, eps=1e-6):
        g, b, m, v = bn if bn is not None else (None, None, None, None)
        self.check(lib().aig_fc_plan_set_weights(self.handle, ptr(w_in_out), ptr(bias), ptr(g), ptr(b), ptr(m), ptr(v), eps))

    def set_weights_out_in(self, w_out_in, bias):
        self.check(lib().aig_fc_plan_set_weights_out_in(self.handle, ptr(w_out_in), ptr(bias)))

    def forward(self, x, y, residual=None):
        self.check(lib().aig_conv_forward(self.handle, ptr(x), ptr(residual), ptr(y)))
        return y


class FcBackwardPlan(_Plan):
    """aig_fc_backward_*: weight, bias and input gradients of a fully connected layer (FCLayer.cpp:54-59)."""
    _destroy = "aig_fc_backward_plan_destroy"

    def __init__(self, ctx, batch, in_c, out_c):
        super().__init__(ctx)
        self.check(lib().aig_fc_backward_plan_create(ctx.handle, batch, in_c, out_c, ctypes.byref(self.handle)))

    def backward(self, x, grad, w_in_out, grad_w=None, grad_b=None, grad_x=None):
        self.check(lib().aig_fc_backward(self.handle, ptr(x), ptr(grad), ptr(w_in_out), ptr(grad_w), ptr(grad_b), ptr(grad_x)))


class Conv0Plan(_Plan):
    """aig_conv0_plan: first-layer (3-channel) convolution with fused input conversion."""
    _destroy = "aig_conv0_plan_destroy"
    _dims = "aig_conv0_plan_out_dims"

    def __init__(self, ctx, batch, in_h, in_w, out_c, k, stride, pad, act=ACT_NONE, slope=0.01, in_d=None, kd=1, sd=1, pd=0):
        super().__init__(ctx)
        if in_d is None:
            self.check(lib().aig_conv0_plan_create(ctx.handle, batch, in_h, in_w, out_c, k, stride, pad, act, slope,
                                                   ctypes.byref(self.handle)))
        else:
            self.check(lib().aig_conv0_plan_create_3d(ctx.handle, batch, in_d, in_h, in_w, out_c, kd, k, sd, stride, pd, pad,
                                                      act, slope, ctypes.byref(self.handle)))

    def set_weights(self, w, bias, bn=None, eps=1e-6):
        g, b, m, v = bn if bn is not None else (None, None, None, None)
        self.check(lib().aig_conv0_plan_set_weights(self.handle, ptr(w), ptr(bias), ptr(g), ptr(b), ptr(m), ptr(v), eps))

    def forward_bgra(self, bgra, y):
        self.check(lib().aig_conv0_forward_bgra(self.handle, ptr(bgra), ptr(y)))
        return y

    def forward_rgb_planar(self, rgb, y):
        self.check(lib().aig_conv0_forward_rgb_planar(self.handle, ptr(rgb), ptr(y)))
        return y

    def forward_nchw(self, x, y):
        self.check(lib().aig_conv0_forward_nchw(self.handle, ptr(x), ptr(y)))
        return y


class CnnEncoder:
    """aig_cnn: the 2-D frame encoder (host C++ runner over the kernel ABI)."""

    def __init__(self, ctx, batch, height, width, widths=(32, 64, 128, 256, 256), k0=5, n_out=18, n_sigmoid=16,
                 act=ACT_SWISH, slope=0.01):
        self.ctx = ctx
        w = (c_int * (AIG_CNN_MAX_BLOCKS + 1))(*widths)
        self.cfg = CnnConfig(batch, height, width, len(widths) - 1, w, k0, n_out, n_sigmoid, act, slope)
        self.handle = c_void_p()
        rc = lib().aig_cnn_create(ctx.handle, ctypes.byref(self.cfg), ctypes.byref(self.handle))
        if rc != 0:
            raise AigError(rc, lib().aig_last_error(ctx.handle).decode())
        self.widths = tuple(widths)

    def check(self, rc):
        if rc != 0:
            raise AigError(rc, lib().aig_cnn_last_error(self.handle).decode())

    def checkpoint_bytes(self):
        return lib().aig_cnn_checkpoint_bytes(ctypes.byref(self.cfg))

    def load_bytes(self, blob):
        buf = (ctypes.c_char * len(blob)).from_buffer_copy(blob)
        self.check(lib().aig_cnn_load_memory(self.handle, ctypes.cast(buf, c_void_p), len(blob)))

    def load_file(self, path):
        self.check(lib().aig_cnn_load_file(self.handle, path.encode()))

    def forward(self, bgra_dev, graph=False):
        fn = lib().aig_cnn_forward_graph if graph else lib().aig_cnn_forward
        self.check(fn(self.handle, ptr(bgra_dev)))

    def forward_rgb(self, rgb_planar_dev, graph=False):
        fn = lib().aig_cnn_forward_graph_rgb if graph else lib().aig_cnn_forward_rgb
        self.check(fn(self.handle, ptr(rgb_planar_dev)))

    def submit_host_rgb(self, slot, rgb_host, out_host):
        self.check(lib().aig_cnn_submit_host_rgb(self.handle, slot, ptr(rgb_host), ptr(out_host)))

    def infer_host(self, bgra_host, out_host):
        self.check(lib().aig_cnn_infer_host(self.handle, ptr(bgra_host), ptr(out_host)))

    def submit_host(self, slot, bgra_host, out_host):
        self.check(lib().aig_cnn_submit_host(self.handle, slot, ptr(bgra_host), ptr(out_host)))

    def wait(self, slot):
        self.check(lib().aig_cnn_wait(self.handle, slot))

    def _view(self, addr, shape, dtype):
        import torch

        n = 1
        for s in shape:
            n *= s
        out = torch.empty(shape, dtype=dtype, device="cuda:%d" % self.ctx.device)
        esz = out.element_size()
        self.ctx.call("aig_memcpy", c_void_p(out.data_ptr()), c_void_p(addr), n * esz)
        self.ctx.sync()
        return out

    def outputs_half(self):
        import torch

        return self._view(lib().aig_cnn_outputs_half(self.handle), (self.cfg.batch, self.cfg.n_out), torch.float16)

    def outputs_f32(self):
        import torch

        return self._view(lib().aig_cnn_outputs_f32(self.handle), (self.cfg.batch, self.cfg.n_out), torch.float32)

    def features(self):
        import torch

        return self._view(lib().aig_cnn_features(self.handle), (self.cfg.batch, self.widths[-1]), torch.float16)

    def stage_output(self, stage):
        import torch

        h, w, c = c_int(), c_int(), c_int()
        addr = lib().aig_cnn_stage_output(self.handle, stage, ctypes.byref(h), ctypes.byref(w), ctypes.byref(c))
        return self._view(addr, (self.cfg.batch, h.value, w.value, c.value), torch.float16)

    @property
    def kernel_launches(self):
        return lib().aig_cnn_kernel_launches(self.handle)

    def profile_begin(self, max_steps):
        self.check(lib().aig_cnn_profile_begin(self.handle, max_steps))

    def profile_end(self):
        """[(site name, mean ms, algorithmic flops, algorithmic bytes)], steps recorded."""
        n = lib().aig_cnn_site_count(self.handle)
        ms = (ctypes.c_double * n)()
        steps = c_int()
        self.check(lib().aig_cnn_profile_end(self.handle, ms, n, ctypes.byref(steps)))
        rows = [(lib().aig_cnn_site_name(self.handle, i).decode(), ms[i], lib().aig_cnn_site_flops(self.handle, i),
                 lib().aig_cnn_site_bytes(self.handle, i)) for i in range(n)]
        return rows, steps.value

    def close(self):
        if self.handle:
            lib().aig_cnn_destroy(self.handle)
            self.handle = c_void_p()


class LstmPlan(_Plan):
    """aig_lstm_plan: hoisted input projection + persistent recurrent kernel."""
    _destroy = "aig_lstm_plan_destroy"

    def __init__(self, ctx, seq_len, layers, hidden, batch, in_c, clip=5.0, double_bias=True, batch_major=False):
        super().__init__(ctx)
        self.check(lib().aig_lstm_plan_create(ctx.handle, seq_len, layers, hidden, batch, in_c, clip, 1 if double_bias else 0,
                                              1 if batch_major else 0, ctypes.byref(self.handle)))

    def set_weights(self, blob):
        self._keep = [blob]
        self.check(lib().aig_lstm_plan_set_weights(self.handle, ptr(blob)))

    def forward(self, x, y, h_state=None, c_state=None, use_state=False):
        self.check(lib().aig_lstm_forward(self.handle, ptr(x), ptr(y), ptr(h_state), ptr(c_state), 1 if use_state else 0))
        return y


class MhaPlan(_Plan):
    """aig_mha_plan: projections + tcgen05 attention tile kernel (+ ring KV cache step)."""
    _destroy = "aig_mha_plan_destroy"

    def __init__(self, ctx, batch, seq_len, embed, heads, rope_base=0.0, window=0):
        super().__init__(ctx)
        self.check(lib().aig_mha_plan_create(ctx.handle, batch, seq_len, embed, heads, rope_base, window, ctypes.byref(self.handle)))

    def set_weights(self, wq, wk, wv, wo):
        self._keep = [wq, wk, wv, wo]
        self.check(lib().aig_mha_plan_set_weights(self.handle, ptr(wq), ptr(wk), ptr(wv), ptr(wo)))

    def forward(self, x, y, pos0=0):
        self.check(lib().aig_mha_forward(self.handle, ptr(x), ptr(y), pos0))
        return y

    def step(self, x, y, position):
        self.check(lib().aig_mha_step(self.handle, ptr(x), ptr(y), position))
        return y

    def reset(self):
        self.check(lib().aig_mha_reset(self.handle))


class Recording:
    """aig_recording: a recording file of the reference's input recorder (int32 width, height; per frame a 10-byte
    input header and a planar RGB uint8 frame)."""

    def __init__(self, path):
        self.handle = c_void_p()
        rc = lib().aig_recording_open(str(path).encode(), ctypes.byref(self.handle))
        if rc != 0:
            raise AigError(rc, lib().aig_recording_last_error(None).decode())
        w, h, n = c_int(), c_int(), ctypes.c_longlong()
        lib().aig_recording_info(self.handle, ctypes.byref(w), ctypes.byref(h), ctypes.byref(n))
        self.width, self.height, self.n_records = w.value, h.value, n.value

    def check(self, rc):
        if rc != 0:
            raise AigError(rc, lib().aig_recording_last_error(self.handle).decode())

    def read(self, first, count):
        """(frames uint8 [count][3][h][w], key_states uint16 [count], mouse int32 [count][2]) as numpy arrays."""
        import numpy as np

        frames = np.empty((count, 3, self.height, self.width), np.uint8)
        keys = np.empty(count, np.uint16)
        mouse = np.empty((count, 2), np.int32)
        self.check(lib().aig_recording_read(self.handle, first, count, ptr(frames), ptr(keys), ptr(mouse)))
        return frames, keys, mouse

    @staticmethod
    def targets(keys, mouse):
        import numpy as np

        keys, mouse = np.ascontiguousarray(keys, np.uint16), np.ascontiguousarray(mouse, np.int32)
        out = np.empty((keys.size, 16), np.float32)
        rc = lib().aig_recording_targets(ptr(keys), ptr(mouse), keys.size, ptr(out))
        if rc != 0:
            raise AigError(rc, "aig_recording_targets")
        return out

    def infer(self, encoder, first, count):
        """Frame encoder outputs [count][n_out] for records first .. first+count-1 (planar RGB straight from the file)."""
        import numpy as np

        out = np.empty((count, encoder.cfg.n_out), np.float32)
        rc = lib().aig_cnn_infer_recording(encoder.handle, self.handle, first, count, encoder.cfg.batch, encoder.cfg.n_out, ptr(out))
        if rc != 0:
            msg = lib().aig_recording_last_error(self.handle).decode() or lib().aig_cnn_last_error(encoder.handle).decode()
            raise AigError(rc, msg)
        return out

    def close(self):
        if self.handle:
            lib().aig_recording_close(self.handle)
            self.handle = c_void_p()
