from wallx_b200.utils.timers import DummyTimer, Timer, Timers  # noqa: F401
