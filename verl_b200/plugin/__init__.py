"""Extension points that live outside the core packages (device platforms)."""
