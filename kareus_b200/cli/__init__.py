"""Command-line drivers: the three phases of a run (profile → compose + plan → execute) and the
comparison tools, with the reference drivers' structure, argument names and output locations
(``tests/artifact/run_kareus.sh``, ``kareus_run_bayesian.sh``, ``create_frontier.sh``,
``compare_method.py``; ``tests/kareus/generate_profile_csv.py``, ``run_optimization.py``)."""
