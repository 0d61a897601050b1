"""Hot ops.  Each function runs a hand-written sm_100a kernel for CUDA tensors and the
plain-PyTorch oracle (``nmoe_b200.ref``) for CPU tensors."""
from .elementwise import embedding, rmsnorm, rope, swiglu, swiglu_bwd_fused
from .tc_gemm import check_status, gemm, grouped_gemm, grouped_wgrad, linear
from .optim import adamw_flat_, sumsq
from .router import router_bias_update_, router_topk
from .attention import attention
from .ce import lm_head_loss
from .quant import dequant_mxfp8, gemm_mxfp8, grouped_gemm_mxfp8, quant_mxfp4, quant_mxfp8, swiglu_quant_mxfp8
