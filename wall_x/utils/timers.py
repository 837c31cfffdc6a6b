from wallx_b200.utils.timers import DummyTimer, Timer, TimerBase, Timers  # noqa: F401
