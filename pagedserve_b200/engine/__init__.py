"""Step function, scheduler, engine entry point and trace replay."""
