from wallx_b200.utils.constant import action_statistic_dof  # noqa: F401
