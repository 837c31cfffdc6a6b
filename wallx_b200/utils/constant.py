"""Per-robot action statistics (``min`` / ``delta`` per DOF group) used for [-1, 1] normalisation.

Same data and same name as the reference's ``wall_x/utils/constant.py:1-362``
(``action_statistic_dof``: 27 robots), stored as a JSON data file next to this module.
"""
import json
import os

with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "robot_stats.json"), "r", encoding="utf-8") as _f:
    action_statistic_dof = json.load(_f)
