"""caminus_b200: the fused per-layer glue kernels of the Caminus inference engine (residual add + RMSNorm, q/k RMSNorm + NeoX
RoPE, SwiGLU + Q8_1 activation quantisation, Q4_K embedding rows) as hand-written CUDA for B200 (sm_100a), behind the
reference's own loader and op-wrapper interface.

    caminus_b200.device.cuda.Module / Kernel     the loader interface of caminus.device.hip
    caminus_b200.prefill.q3m_ops.Ops             emb / add_rms16 / swiglu / qk_rope
    caminus_b200.prefill.q35own.Ops              add_rms16 for any row length
    caminus_b200.engine.gguf                     quantize_q8_1 / silu_mul / swiglu_q8_1
    caminus_b200.glue                            the fp16-storage forms and the per-layer sequence
    caminus_b200.dist                            row sharding and the tensor-parallel RMSNorm

The CUDA library is required: nothing here computes on the CPU or through PyTorch operators."""
__version__ = '0.1.0'
