from minisgl.server.launch import launch_server

if __name__ == "__main__":
    launch_server()
