from .batch import StepBatch, StepEntry, build_batch
from .generate import GenResult, GenStats, GenerationLoop, fit_prompt, plan_batches
from .model import Model, build_plan, load_model, parse_dtype
from .stepper import ModelStepper

__all__ = ["StepBatch", "StepEntry", "build_batch", "GenResult", "GenStats", "GenerationLoop", "fit_prompt",
           "plan_batches", "Model", "build_plan", "load_model", "parse_dtype", "ModelStepper"]
