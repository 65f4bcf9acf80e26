"""Small shared helpers: device timing (``timing``) and repository invariants (``ci_checks``)."""
