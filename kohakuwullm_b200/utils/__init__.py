from kohakuwullm_b200.utils.misc import (  # noqa: F401
    autofill_schedule_steps,
    count_active_parameters,
    count_parameters,
    human_count,
    import_class,
)
