from .dist import BACKEND_NAME, init_process_group, register_backend  # noqa: F401
