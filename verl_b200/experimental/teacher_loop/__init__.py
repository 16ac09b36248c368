"""Distillation teachers served by rollout servers of their own: fleet manager and the scoring client the trainer uses."""

from .teacher_manager import AsyncTeacherLLMServerManager, pad_teacher_outputs, teacher_sampling_params  # noqa: F401
from .teacher_model import TeacherModelManager, TeacherModelSpec, build_teacher_fleet  # noqa: F401
