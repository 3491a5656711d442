"""Step function, scheduler and the generation engine."""
from .batch import StepBatch, StepEntry, build_batch
from .scheduler import AdmissionError, Request, Scheduled, Scheduler
from .step import OutOfPages, StepError, run_step

__all__ = ["StepBatch", "StepEntry", "build_batch", "OutOfPages", "StepError", "run_step", "AdmissionError", "Request",
           "Scheduled", "Scheduler"]
