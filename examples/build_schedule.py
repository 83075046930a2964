"""Build JSON order directives for common pipeline schedules (re-exported from the package)."""
from piper_b200.compiler.builders import (build_1f1b_schedule, build_dualpipev_schedule,  # noqa: F401
                                          build_interleaved_1f1b_schedule, build_zerobubble_schedule, format_rows)


def main() -> None:
    from test_harness import main as harness_main

    harness_main()


if __name__ == "__main__":
    main()
