"""Plan files (schedules and frequencies), the per-microbatch comm scheduler and frontier sampling."""
from .schedule import (CommConfig, ScheduleItem, TRAIL_CONFIG, DEFAULT_CONFIG, parse_config_string,
                       parse_schedule_file, parse_schedule_text, emit_schedule_text, read_trailer,
                       uniform_schedule, FWD_KEYS_TP, BWD_KEYS_TP, FWD_KEYS_CP, BWD_KEYS_CP)
from .freqs import parse_freqs_file, parse_freqs_text, emit_freqs_text, uniform_freqs
from .comm_scheduler import PipelineCommScheduler
from .frontier import sample_frontier, select_max_throughput, create_frontier
