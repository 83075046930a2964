from ._core import ActorDiedError, GetTimeoutError, RayActorError, RayError, RayTaskError  # noqa: F401
