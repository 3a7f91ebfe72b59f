"""Stand-alone operator wrappers named after the reference's kernel holders:

    RoPEKernel        Sources/EdgeRunnerMetal/RoPEKernel.swift:4-307     (execute / encodeNeoX)
    GQAKernel         Sources/EdgeRunnerMetal/GQAKernel.swift:4-187      (execute / encode on fp16 K/V)
    TurboQuantKernel  Sources/EdgeRunnerMetal/TurboQuantKernel.swift:13-112 (quantize rows)
    Gemma4DecodeKernels  Sources/EdgeRunnerMetal/Gemma4DecodeKernels.swift:537-660 (runDecodeGQAF16KVWindowed only)

`encode*` methods enqueue on a stream with device buffers (the command-buffer style of the reference);
`execute*` methods are the array-in / array-out convenience forms used by the reference's tests.
"""
import ctypes as C
import math

import numpy as np

from ._lib import ERGQAParams, ERRoPEParams, ERWindowedGQAParams, check, lib, ptr, stream_ptr


def _torch():
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("edgerunner_b200 operators need a CUDA device (no CPU fallback)")
    return torch


class RoPEKernel:
    def encode_neox(self, input_buffer, output_buffer, seq_len, num_heads, head_dim, start_pos=0, theta=10000.0,
                    scaling_factor=1.0, partial_rotary_factor=1.0, to_f16=False, stream=None):
        p = ERRoPEParams(seq_len, num_heads, head_dim, start_pos, theta, scaling_factor, partial_rotary_factor)
        fn = lib().er_rope_neox_f32_to_f16 if to_f16 else lib().er_rope_neox_f32
        check(fn(ptr(input_buffer), ptr(output_buffer), C.byref(p), stream_ptr(stream)))

    def execute_neox(self, input, seq_len, num_heads, head_dim, start_pos=0, theta=10000.0, scaling_factor=1.0,
                     partial_rotary_factor=1.0, to_f16=False):
        torch = _torch()
        x = torch.as_tensor(np.ascontiguousarray(input, dtype=np.float32)).cuda()
        out = torch.empty(x.shape, dtype=torch.float16 if to_f16 else torch.float32, device="cuda")
        self.encode_neox(x, out, seq_len, num_heads, head_dim, start_pos, theta, scaling_factor, partial_rotary_factor, to_f16)
        torch.cuda.synchronize()
        return out.cpu().numpy()


class GQAKernel:
    block_size = 16                 # GQAKernel.blockSize
    max_optimized_head_dim = 128    # GQAKernel.maxOptimizedHeadDim

    max_supported_head_dim = 512    # GQAKernel.maxSupportedHeadDim

    def encode_f32(self, q_buffer, k_buffer, v_buffer, output_buffer, seq_len, head_dim, num_heads, num_kv_heads, causal,
                   kv_seq_len=0, q_offset=0, additive_mask_buffer=None, stream=None):
        """GQAKernel.encode (GQAKernel.swift:113-172): float32 q/k/v/out device buffers, optional additive mask
        [seq_len, kv_seq_len] (-inf hides a key)."""
        p = ERGQAParams(seq_len, head_dim, num_heads, num_kv_heads, num_heads // num_kv_heads, 1.0 / math.sqrt(head_dim),
                        int(bool(causal)), self.block_size, self.block_size, kv_seq_len, q_offset)
        check(lib().er_gqa_attention_f32(ptr(q_buffer), ptr(k_buffer), ptr(v_buffer), ptr(output_buffer),
                                         ptr(additive_mask_buffer), C.byref(p), stream_ptr(stream)))

    def execute(self, q, k, v, seq_len, head_dim, num_heads, num_kv_heads, causal, kv_seq_len=0, q_offset=0, additive_mask=None):
        """GQAKernel.execute (GQAKernel.swift:27-110): arrays in, array out."""
        torch = _torch()
        eff = kv_seq_len if kv_seq_len > 0 else seq_len
        qd = torch.as_tensor(np.ascontiguousarray(q, dtype=np.float32)).cuda()
        kd = torch.as_tensor(np.ascontiguousarray(k, dtype=np.float32)).cuda()
        vd = torch.as_tensor(np.ascontiguousarray(v, dtype=np.float32)).cuda()
        assert qd.numel() == seq_len * num_heads * head_dim and kd.numel() == vd.numel() == eff * num_kv_heads * head_dim
        md = None
        if additive_mask is not None:
            md = torch.as_tensor(np.ascontiguousarray(additive_mask, dtype=np.float32)).cuda()
            assert md.numel() == seq_len * eff
        out = torch.empty_like(qd)
        self.encode_f32(qd, kd, vd, out, seq_len, head_dim, num_heads, num_kv_heads, causal, kv_seq_len, q_offset, md)
        torch.cuda.synchronize()
        return out.cpu().numpy()

    def encode(self, q_buffer, k_buffer, v_buffer, output_buffer, seq_len, head_dim, num_heads, num_kv_heads, causal,
               kv_seq_len=0, q_offset=0, scale=None, stream=None):
        """fp16 K/V variant (pipelineF16KV): q/out float32 [S,H,D], k/v float16 [T,Hkv,D] device buffers."""
        p = ERGQAParams(seq_len, head_dim, num_heads, num_kv_heads, num_heads // num_kv_heads,
                        (1.0 / math.sqrt(head_dim)) if scale is None else scale, int(bool(causal)), self.block_size,
                        self.block_size, kv_seq_len, q_offset)
        check(lib().er_gqa_attention_f16kv(ptr(q_buffer), ptr(k_buffer), ptr(v_buffer), ptr(output_buffer), C.byref(p),
                                           stream_ptr(stream)))

    def encode_static_workspace(self, q_buffer, k_buffer, v_buffer, output_buffer, seq_len, head_dim, num_heads, num_kv_heads,
                                causal, kv_seq_len=0, q_offset=0, scale=None, stream=None):
        """Same operator through er_gqa_attention_f16kv_static: for hosts where the library must not allocate device
        memory (the workspace is a ~1 MiB array inside the library; at most 16 kv heads, group size 1/2/4)."""
        p = ERGQAParams(seq_len, head_dim, num_heads, num_kv_heads, num_heads // num_kv_heads,
                        (1.0 / math.sqrt(head_dim)) if scale is None else scale, int(bool(causal)), self.block_size,
                        self.block_size, kv_seq_len, q_offset)
        check(lib().er_gqa_attention_f16kv_static(ptr(q_buffer), ptr(k_buffer), ptr(v_buffer), ptr(output_buffer), C.byref(p),
                                                  stream_ptr(stream)))

    def execute_f16kv(self, q, k, v, seq_len, head_dim, num_heads, num_kv_heads, causal, kv_seq_len=0, q_offset=0):
        torch = _torch()
        qd = torch.as_tensor(np.ascontiguousarray(q, dtype=np.float32)).cuda()
        kd = torch.as_tensor(np.ascontiguousarray(k, dtype=np.float16)).cuda()
        vd = torch.as_tensor(np.ascontiguousarray(v, dtype=np.float16)).cuda()
        out = torch.empty_like(qd)
        self.encode(qd, kd, vd, out, seq_len, head_dim, num_heads, num_kv_heads, causal, kv_seq_len, q_offset)
        torch.cuda.synchronize()
        return out.cpu().numpy()


class Gemma4DecodeKernels:
    """The sliding-window decode attention of the Gemma 4 kernel holder; its other kernels are outside this backend."""

    def encode_decode_gqa_f16kv_windowed(self, q_buffer, key_cache_buffer, value_cache_buffer, output_buffer, num_heads,
                                         num_kv_heads, head_dim, kv_start, kv_count, kv_capacity, attention_scale=None,
                                         stream=None):
        p = ERWindowedGQAParams(num_heads, num_kv_heads, head_dim, kv_start, kv_count, kv_capacity,
                                0.0 if attention_scale is None else attention_scale)
        check(lib().er_gqa_attention_f16kv_windowed(ptr(q_buffer), ptr(key_cache_buffer), ptr(value_cache_buffer),
                                                    ptr(output_buffer), C.byref(p), stream_ptr(stream)))

    def run_decode_gqa_f16kv_windowed(self, q, k, v, num_heads, num_kv_heads, head_dim, kv_start, kv_count, kv_capacity,
                                      attention_scale=None):
        torch = _torch()
        qd = torch.as_tensor(np.ascontiguousarray(q, dtype=np.float32)).cuda()
        kd = torch.as_tensor(np.ascontiguousarray(k, dtype=np.float16)).cuda()
        vd = torch.as_tensor(np.ascontiguousarray(v, dtype=np.float16)).cuda()
        assert qd.numel() == num_heads * head_dim and kd.numel() == vd.numel() == kv_capacity * num_kv_heads * head_dim
        out = torch.empty_like(qd)
        self.encode_decode_gqa_f16kv_windowed(qd, kd, vd, out, num_heads, num_kv_heads, head_dim, kv_start, kv_count,
                                              kv_capacity, attention_scale)
        torch.cuda.synchronize()
        return out.cpu().numpy()


class TurboQuantKernel:
    def encode_quantize_rows(self, source, row_count, source_row_stride, destination_row_base, bits, out_codes,
                             out_residual_signs, out_outlier_mask, out_metadata, stream=None):
        check(lib().er_turboquant_quantize_rows(ptr(source), row_count, source_row_stride, destination_row_base, bits,
                                                ptr(out_codes), ptr(out_residual_signs), ptr(out_outlier_mask),
                                                ptr(out_metadata), stream_ptr(stream)))

    PRESETS = {"balanced": (3, 5, 32), "aggressive": (2, 3, 32)}   # TurboQuantPreset.descriptor (TurboQuant.swift:78-84, 117-124)

    def encode_quantize_rows_outliers(self, source, row_count, source_row_stride, destination_row_base, regular_bits, high_bits,
                                      high_count, use_quantization_benefit, out_codes, out_residual_signs, out_outlier_mask,
                                      out_metadata, stream=None):
        check(lib().er_turboquant_quantize_rows_outliers(ptr(source), row_count, source_row_stride, destination_row_base, regular_bits,
                                                         high_bits, high_count, int(bool(use_quantization_benefit)), ptr(out_codes),
                                                         ptr(out_residual_signs), ptr(out_outlier_mask), ptr(out_metadata),
                                                         stream_ptr(stream)))

    def execute_quantize_rows_preset(self, rows, preset, use_quantization_benefit=False):
        """rows: [n, >=128] float32, preset "balanced" | "aggressive" -> (codes [n,w] u32, signs [n,4], mask [n,4], meta [n,2])."""
        torch = _torch()
        rb, hb, cnt = self.PRESETS[preset]
        x = torch.as_tensor(np.ascontiguousarray(rows, dtype=np.float32)).cuda()
        n, stride = x.shape
        w = (128 * rb + 31) // 32 + (cnt * (hb - rb) + 31) // 32
        codes = torch.full((n, w), -1, dtype=torch.int32, device="cuda")
        signs = torch.full((n, 4), -1, dtype=torch.int32, device="cuda")
        mask = torch.full((n, 4), -1, dtype=torch.int32, device="cuda")
        meta = torch.full((n, 2), float("nan"), dtype=torch.float32, device="cuda")
        self.encode_quantize_rows_outliers(x, n, stride, 0, rb, hb, cnt, use_quantization_benefit, codes, signs, mask, meta)
        torch.cuda.synchronize()
        return (codes.cpu().numpy().view(np.uint32), signs.cpu().numpy().view(np.uint32),
                mask.cpu().numpy().view(np.uint32), meta.cpu().numpy())

    def execute_quantize_rows(self, rows, bits):
        """rows: [n, >=128] float32 -> (codes [n,w] u32, signs [n,4], mask [n,4], meta [n,2])."""
        torch = _torch()
        x = torch.as_tensor(np.ascontiguousarray(rows, dtype=np.float32)).cuda()
        n, stride = x.shape
        w = (128 * bits + 31) // 32
        codes = torch.full((n, w), -1, dtype=torch.int32, device="cuda")
        signs = torch.full((n, 4), -1, dtype=torch.int32, device="cuda")
        mask = torch.full((n, 4), -1, dtype=torch.int32, device="cuda")
        meta = torch.full((n, 2), float("nan"), dtype=torch.float32, device="cuda")
        self.encode_quantize_rows(x, n, stride, 0, bits, codes, signs, mask, meta)
        torch.cuda.synchronize()
        return (codes.cpu().numpy().view(np.uint32), signs.cpu().numpy().view(np.uint32),
                mask.cpu().numpy().view(np.uint32), meta.cpu().numpy())


class Q8Kernel:
    """quantize_q8_0_rows (Shaders/Dequant_Q8_0.metal:19-49) on device buffers."""

    def encode_quantize_rows(self, source, row_count, source_row_stride, destination_row_base, destination_blocks, stream=None):
        check(lib().er_quantize_q8_0_rows(ptr(source), row_count, source_row_stride, destination_row_base, ptr(destination_blocks),
                                          stream_ptr(stream)))

    def execute_quantize_rows(self, rows):
        """rows: [n, >=128] float32 -> uint8 [n, 136] (four 34-byte blocks per row)."""
        torch = _torch()
        x = torch.as_tensor(np.ascontiguousarray(rows, dtype=np.float32)).cuda()
        n, stride = x.shape
        out = torch.full((n, 136), 0xEE, dtype=torch.uint8, device="cuda")
        self.encode_quantize_rows(x, n, stride, 0, out)
        torch.cuda.synchronize()
        return out.cpu().numpy()
