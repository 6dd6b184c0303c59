from .launch import run_ranks  # noqa: F401
