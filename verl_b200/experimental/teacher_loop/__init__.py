from .teacher_manager import AsyncTeacherLLMServerManager  # noqa: F401
from .teacher_model import MultiTeacherModelManager, TeacherModelManager, TeacherServer  # noqa: F401
