"""Extension points for code that lives outside this package."""
