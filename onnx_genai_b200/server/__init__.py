from .app import EngineDriver, create_app  # noqa: F401
