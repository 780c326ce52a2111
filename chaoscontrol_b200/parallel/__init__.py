from .distributed import (AsyncGradAllReducer, allreduce_grads, broadcast_params,
                          clip_arena_grad_norm, clip_grad_norm_fused, resolve_ddp_context,
                          should_stop_now)

__all__ = ["AsyncGradAllReducer", "allreduce_grads", "broadcast_params", "clip_arena_grad_norm",
           "clip_grad_norm_fused", "resolve_ddp_context", "should_stop_now"]
