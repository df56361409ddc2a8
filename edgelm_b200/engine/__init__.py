from .generate import Generation, GenerationError, GenerationLoop, GenerationStats, plan_batches

__all__ = ["Generation", "GenerationError", "GenerationLoop", "GenerationStats", "plan_batches"]
